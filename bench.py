#!/usr/bin/env python
"""Decode benchmark of the Qwen3-32B-shaped Q8_0 layer stack (batch 1).

One step = one decoded token through 64 layers x (Q|K|V 10240x5120, o_proj
5120x8192, gate/up 25600x5120, down 5120x25600) + LM head 151936x5120, all
Q8_0 with random-initialised weights (a seeded on-device generator stands in
for a model file; 33.98 GB of distinct weight bytes, far larger than L2), the
attention core replaced by the identity on the roped Q slice.

  python bench.py --gpus N --steps K --warmup W            # this library
  python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU path

With N > 1 (torchrun, one rank per GPU) the weights are sharded per matvec
(column-parallel Q|K|V, gate/up and LM head; row-parallel o_proj and down) and
partial sums are combined with NCCL over NVLink; the same token is decoded, so
scaling is strong.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import mmap
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, N_HEADS, N_KV, HEAD_DIM, FFN, VOCAB, N_LAYERS = 5120, 64, 8, 128, 25600, 151936, 64
EPS, ROPE_BASE = 1e-6, 1e6
Q8_0 = 8
FALLBACK_HBM_GBS = 6650.0


def q8_bytes(n_out, n_in):
    return n_out * (n_in // 32) * 34


def ty_bytes(ty, n_out, n_in):
    return q8_bytes(n_out, n_in) if ty == Q8_0 else n_out * (n_in // 256) * 144


def layer_tensors(hidden, nq, nkv, ffn):
    return [("wq", nq, hidden), ("wk", nkv, hidden), ("wv", nkv, hidden), ("wo", hidden, nq),
            ("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn)]


def rope_table(pos, rot_dim, base):
    i = np.arange(rot_dim // 2, dtype=np.float32)
    inv = np.power(np.float32(base), (np.float32(-2.0) * i / np.float32(rot_dim)).astype(np.float32)).astype(np.float32)
    t = (np.float32(pos) * inv).astype(np.float32)
    return np.stack([np.sin(t), np.cos(t)], axis=1).astype(np.float32)[None]


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def ncu_traffic():
    """Per-token DRAM bytes of the matvec kernel from the committed ncu capture, if any."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            return json.load(f)
    except Exception:
        return None


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in open(self.path):
            f = [v.strip() for v in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower() == "active":
                    reasons.add(n)
        os.unlink(self.path)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_setup(world):
    if world == 1:
        return None
    import torch.distributed as dist

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group(backend="gloo")  # host-side plumbing only; the data path is NCCL inside the library
    return dist


def build_model(g, n_layers, write_host_layers, rank, ty=Q8_0, m=1, head=True):
    """Reserve a host mapping for the whole model, attach it, and fill the
    tensors from the on-device generator (seeds 2000 + 8*layer + k)."""
    from allpaka_b200 import gpu as G
    from allpaka_b200 import synth

    nq, nkv = N_HEADS * HEAD_DIM, N_KV * HEAD_DIM
    specs = layer_tensors(HIDDEN, nq, nkv, FFN)
    vocab = VOCAB if head else 1024
    off, offsets = 0, []
    for _ in range(n_layers):
        lo = {}
        for name, n_out, n_in in specs:
            lo[name] = off
            off += (ty_bytes(ty, n_out, n_in) + 255) // 256 * 256
        offsets.append(lo)
    head_off = off
    off += (ty_bytes(ty, vocab, HIDDEN) + 255) // 256 * 256
    mm = mmap.mmap(-1, off, flags=mmap.MAP_PRIVATE | mmap.MAP_ANONYMOUS | getattr(mmap, "MAP_NORESERVE", 0))
    region = np.frombuffer(mm, dtype=np.uint8)
    assert g.attach(region)
    layers, host = [], {}
    for l in range(n_layers):
        views = {}
        for k, (name, n_out, n_in) in enumerate(specs):
            v = region[offsets[l][name]: offsets[l][name] + ty_bytes(ty, n_out, n_in)]
            g.synth_matrix(v, ty, n_out, n_in, 2000 + 8 * l + k, write_host=(l in write_host_layers))
            views[name] = v
        an, fn = synth.gamma(HIDDEN, 5000 + 2 * l), synth.gamma(HIDDEN, 5001 + 2 * l)
        layers.append(G.TokenLayer(an, fn, (ty, views["wq"], nq), (ty, views["wk"], nkv),
                                   (ty, views["wv"], nkv), (ty, views["wo"], HIDDEN),
                                   (ty, views["gate"], FFN), (ty, views["up"], FFN),
                                   (ty, views["down"], HIDDEN)))
        if l in write_host_layers:
            host[l] = dict(views, attn_norm=an, ffn_norm=fn)
    hd = region[head_off: head_off + ty_bytes(ty, vocab, HIDDEN)]
    g.synth_matrix(hd, ty, vocab, HIDDEN, 1999, write_host=bool(write_host_layers))
    out_norm = synth.gamma(HIDDEN, 4999)
    x = synth.normal_f32((m, HIDDEN), 4242)
    pos0 = int(np.random.default_rng(4243).integers(0, 32768 - 8))
    rope = np.concatenate([rope_table(pos0 + i, HEAD_DIM, ROPE_BASE) for i in range(m)])
    req = G.TokenReq(layers, out_norm, (ty, hd, vocab), x, m, rope, HEAD_DIM, EPS, HIDDEN, HEAD_DIM,
                     N_HEADS, N_KV)
    return req, host, hd, out_norm, (mm, region)


def token_bytes(n_layers, world=1):
    """Algorithmic bytes of one decoded token: original GGUF weight bytes, f32
    activations in, f32 results out, norm weights and the RoPE table."""
    nq, nkv = N_HEADS * HEAD_DIM, N_KV * HEAD_DIM
    per_layer_w = sum(q8_bytes(o, i) for _, o, i in layer_tensors(HIDDEN, nq, nkv, FFN))
    per_layer_io = (HIDDEN + nq + 2 * nkv) * 4 + (nq + HIDDEN) * 4 + (HIDDEN + FFN) * 4 + (FFN + HIDDEN) * 4 \
        + 2 * HIDDEN * 4 + 512
    return n_layers * (per_layer_w + per_layer_io) + q8_bytes(VOCAB, HIDDEN) + (HIDDEN * 2 + VOCAB) * 4


def cpu_pass(orc, host, head, out_norm, req):
    """One pass of the reference's CPU path (oracle restatement) over layer 0 and
    the LM head with all host threads; returns (layer seconds, head seconds)."""
    nq, nkv = N_HEADS * HEAD_DIM, N_KV * HEAD_DIM
    x = np.array(req.x, dtype=np.float32).reshape(-1)
    rope = np.asarray(req.rope, dtype=np.float32).reshape(-1, 2)
    t0 = time.perf_counter()
    xo = orc.decode_layers(Q8_0, [host[0]], HIDDEN, nq, nkv, HEAD_DIM, FFN, EPS, rope, x, threads=0)
    t1 = time.perf_counter()
    orc.lm_head(Q8_0, head, VOCAB, HIDDEN, xo, out_norm, EPS, threads=0)
    return t1 - t0, time.perf_counter() - t1


def cpu_reference_sample(host, head, out_norm, req, budget_s):
    from oracle import oracle as orc

    orc.build()
    cpu_pass(orc, host, head, out_norm, req)  # warm: page in the weights, start the threads
    tl, th = [], []
    t_start = time.perf_counter()
    while len(tl) < 3 or (time.perf_counter() - t_start < budget_s and len(tl) < 50):
        a, b = cpu_pass(orc, host, head, out_norm, req)
        tl.append(a)
        th.append(b)
    return {"t_layer_s": float(np.median(tl)), "t_head_s": float(np.median(th)), "cores": orc.cpu_threads(),
            "reps": len(tl)}


def host_model_sample():
    """Layer 0 + LM head in host memory.  The bytes come from the library's
    on-device generator when a GPU is present, else from numpy; either way the
    timed work of the reference arm is CPU only."""
    from allpaka_b200 import synth

    try:
        from allpaka_b200 import gpu as G

        g = G.Gpu(0)
        req, host, head, out_norm, keep = build_model(g, 1, {0}, 0)
        g.synth_release()
        g.close()
        return req, host, head, out_norm, keep
    except Exception:
        nq, nkv = N_HEADS * HEAD_DIM, N_KV * HEAD_DIM
        rng = np.random.default_rng(2000)
        host = {0: {}}
        for name, n_out, n_in in layer_tensors(HIDDEN, nq, nkv, FFN):
            w = rng.integers(0, 256, size=q8_bytes(n_out, n_in), dtype=np.uint8)
            host[0][name] = synth.tame_scales(w, Q8_0)
        host[0]["attn_norm"], host[0]["ffn_norm"] = synth.gamma(HIDDEN, 5000), synth.gamma(HIDDEN, 5001)
        head = synth.tame_scales(rng.integers(0, 256, size=q8_bytes(VOCAB, HIDDEN), dtype=np.uint8), Q8_0)

        class R:
            x = synth.normal_f32((1, HIDDEN), 4242)
            rope = rope_table(1234, HEAD_DIM, ROPE_BASE)

        return R, host, head, synth.gamma(HIDDEN, 4999), None


def run_reference(args, rank, world):
    if rank != 0:
        return
    from oracle import oracle as orc

    orc.build()
    req, host, head, out_norm, keep = host_model_sample()
    for _ in range(max(1, args.warmup)):
        cpu_pass(orc, host, head, out_norm, req)
    steps = [cpu_pass(orc, host, head, out_norm, req) for _ in range(args.steps)]
    tl = float(np.median([s[0] for s in steps]))
    th = float(np.median([s[1] for s in steps]))
    t_tok = N_LAYERS * tl + th
    val = 1.0 / t_tok
    line = {
        "impl": "reference", "metric": "decode tok/s Qwen3-32B-shape Q8_0", "value": val, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_tok * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 x int8 -> int32, f32 scales",
        "data": "synthetic",
        "config": {"workload": "qwen3-32b-shaped decode step, 64 layers + lm_head, Q8_0, batch 1",
                   "timed": "CPU restatement of the reference path; each step = layer 0 + lm_head; "
                            "token time = 64 x layer + head"},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": orc.cpu_threads(), "kind": "port",
                         "sample": "1 of 64 layers (518 MB of Q8_0 weights) + lm_head (826 MB) per step",
                         "gbs": token_bytes(N_LAYERS) / t_tok / 1e9},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank, world, local_rank):
    from allpaka_b200 import gpu as G

    dist = dist_setup(world)
    g = G.Gpu(local_rank)
    if world > 1:
        ids = [G.Gpu.dist_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        g.dist_init(rank, world, ids[0])
        if args.tp_exchange == "p2p":
            handles = [None] * world
            dist.all_gather_object(handles, g.p2p_export())
            g.p2p_open(handles)
    n_layers = args.layers
    want_cpu = rank == 0 and world == 1 and not args.no_cpu_baseline
    t_setup = time.perf_counter()
    req, host, head, out_norm, keep = build_model(g, n_layers, {0} if want_cpu else set(), rank)
    g.decode_replay(req, 1)  # uploads + repacks every shard, captures the token graph
    g.synth_release()
    setup_s = time.perf_counter() - t_setup

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v):
        if dist is None:
            return v
        import torch

        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    # ---- device-resident number: K graph replays between one CUDA-event pair
    barrier()
    if args.warmup:
        g.decode_replay(req, args.warmup)
    launches0 = g.stats()[1]
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    ms = g.decode_replay(req, args.steps)   # syncs, records, replays K times, records, syncs
    barrier()
    clocks = sampler.stop()
    gpu_launches = g.stats()[1] - launches0
    ms = max_over_ranks(ms)
    ms_per_step = ms / args.steps
    value = 1e3 / ms_per_step

    # ---- end to end through the public call: host x in, host logits out, every step
    import torch

    xh = torch.empty((1, HIDDEN), dtype=torch.float32).pin_memory()
    xh.numpy()[:] = np.asarray(req.x, dtype=np.float32)
    req.x = xh.numpy()
    for _ in range(max(3, args.warmup)):
        g.decode_token_checked(req)
    barrier()
    torch.cuda.synchronize(local_rank)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        logits = g.decode_token_checked(req)
    torch.cuda.synchronize(local_rank)
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    e2e_val = args.steps / e2e_s
    rope_bytes = int(np.asarray(req.rope).nbytes)

    # ---- roofline of the dominant kernel (the stream-K matvec), timed live per kind
    prof = g.decode_profile(req, reps=3)
    n_launch = {"qkv": n_layers, "wo": n_layers, "gate_up": n_layers, "down": n_layers, "lm_head": 1}
    mv_bytes = sum(prof[k]["bytes"] * n_launch[k] for k in prof)
    mv_ms = sum(prof[k]["ms"] * n_launch[k] for k in prof)
    peak, peak_kind = measured_peak()
    achieved = mv_bytes / (mv_ms * 1e-3) / 1e9
    traffic = ncu_traffic()
    total_launch = sum(n_launch.values())
    roofline = {
        "bound": "hbm", "kernel": "matvec_streamk_kernel<Q8_0, m=1>",
        "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
        "bytes_per_launch": mv_bytes / total_launch, "ms_per_launch": mv_ms / total_launch,
        "launches_per_step": total_launch,
        "traffic": (traffic or {}).get("dram_bytes_per_launch"),
        "by_shape": {k: {"ms": prof[k]["ms"], "gbs": prof[k]["bytes"] / (prof[k]["ms"] * 1e-3) / 1e9} for k in prof},
        "step_frac_of_peak": token_bytes(n_layers) / world / (ms_per_step * 1e-3) / 1e9 / peak,
    }

    cpu = None
    if want_cpu:
        s = cpu_reference_sample(host, head, out_norm, req, args.cpu_budget)
        t_tok = N_LAYERS * s["t_layer_s"] + s["t_head_s"]
        cpu = {"value": 1.0 / t_tok, "unit": "tok/s", "cores": s["cores"], "kind": "port",
               "sample": f"layer 0 + lm_head on host, {s['reps']} timed passes, token time = 64 x layer + head",
               "gbs": token_bytes(N_LAYERS) / t_tok / 1e9}

    if rank == 0:
        line = {
            "metric": "decode tok/s Qwen3-32B-shape Q8_0", "value": value, "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
            "config": {"workload": f"qwen3-32b-shaped decode step, {n_layers} layers + lm_head, Q8_0, batch 1",
                       "weights_gb": token_bytes(n_layers) / 1e9, "l2": "inputs larger than L2 (33.98 GB streamed per step)",
                       "parallelism": ("tp%d, %s reductions" % (world, args.tp_exchange)) if world > 1 else "single gpu",
                       "attention_core": "identity on the roped Q slice"},
            "hbm_gbs": token_bytes(n_layers) / (ms_per_step * 1e-3) / 1e9,
            "e2e": {"value": e2e_val, "unit": "tok/s", "h2d_bytes_per_step": HIDDEN * 4 + rope_bytes,
                    "d2h_bytes_per_step": VOCAB * 4},
            "gpu_launches": int(gpu_launches),
            "roofline": roofline,
            "cpu_baseline": cpu,
            "clocks": clocks,
            "setup_s": setup_s,
        }
        print(json.dumps(line), flush=True)
    barrier()
    g.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=N_LAYERS, help="fewer layers only for quick checks")
    ap.add_argument("--cpu-budget", type=float, default=12.0, help="seconds of CPU-baseline work")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tp-exchange", default="p2p", choices=["p2p", "nccl"],
                    help="how the two per-layer reductions cross GPUs: peer-memory stores or NCCL all-reduce")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()

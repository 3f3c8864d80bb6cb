"""Tensor-parallel decode on 2 GPUs against the single-device oracle (needs >= 2 GPUs; skipped otherwise).

Two child processes, one GPU each, join an NCCL group through the library
(apk_dist_init), upload only their shards and decode the same token; rank 0's
logits must match the CPU oracle of the unsharded model."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ty, m, exchange, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    from allpaka_b200 import gpu as G
    from allpaka_b200 import synth
    from oracle import oracle as orc
    from tests.util import Region, make_layer, oracle_decode, oracle_logits, rel_l2, rope_table

    g = G.Gpu(rank)
    ids = [G.Gpu.dist_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    g.dist_init(rank, world, ids[0])
    if exchange == "p2p":
        handles = [None] * world
        dist.all_gather_object(handles, g.p2p_export())
        g.p2p_open(handles)
    hidden, nh, nkv, ffn, vocab, hd = 1024, 8, 2, 2048, 1536, 128
    nq, nk = nh * hd, nkv * hd
    layers = [make_layer(ty, hidden, nq, nk, ffn, 300 + 100 * l, True) for l in range(2)]
    head = synth.matrix(ty, vocab, hidden, 999)
    names = ("wq", "wk", "wv", "wo", "gate", "up", "down")
    r = Region([L[n] for L in layers for n in names] + [head])
    assert g.attach(r.buf)
    tls = []
    for li, L in enumerate(layers):
        v = dict(zip(names, r.views[li * 7:(li + 1) * 7]))
        tls.append(G.TokenLayer(L["attn_norm"], L["ffn_norm"], (ty, v["wq"], nq), (ty, v["wk"], nk), (ty, v["wv"], nk),
                                (ty, v["wo"], hidden), (ty, v["gate"], ffn), (ty, v["up"], ffn), (ty, v["down"], hidden),
                                L["q_norm"], L["k_norm"]))
    out_norm = synth.gamma(hidden, 998)
    # Four input seeds, none picked.  Chained over layers the f32 additions run in another order
    # than the oracle's (per rank, then across ranks), so a residual value may differ in its last
    # bit; where it sits within an ulp of a .5 rounding boundary one Q8 code flips and moves the
    # logits by ~7e-4 per layer from there on (the single-GPU tests trace such cases to the code).
    # Per seed the figure is recorded; the median must be at rounding level and at most one seed
    # may sit above the chained bar.
    rope = rope_table(orc, np.arange(m) + 4000, hd, hd)
    errs, same, argmax_ok = [], True, True
    for seed in (996, 997, 998, 999):
        x = synth.normal_f32((m, hidden), seed)
        req = G.TokenReq(tls, out_norm, (ty, r.views[-1], vocab), x, m, rope, hd, 1e-6, hidden, hd, nh, nkv)
        logits = g.decode_token_checked(req)
        again = g.decode_token_checked(req)
        req.argmax = True
        ids_ = g.decode_token_checked(req)
        ids_ = ids_.argmax if m > 1 else ids_
        if rank == 0:
            xo = oracle_decode(orc, ty, layers, hidden, nq, nk, hd, ffn, 1e-6, rope, x, m)
            want = oracle_logits(orc, ty, head, vocab, hidden, xo, out_norm, 1e-6, m)
            errs.append(rel_l2(logits, want))
            same = same and bool(np.array_equal(logits, again))
            argmax_ok = argmax_ok and [int(i) for i in ids_] == [int(np.flatnonzero(row == row.max())[-1]) for row in logits]
    if rank == 0:
        out_q.put((errs, same, argmax_ok))
    dist.barrier()
    g.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["nccl", "p2p"])
@pytest.mark.parametrize("ty,m", [(8, 1), (8, 3), (12, 1)])
def test_two_gpu_decode_matches_the_unsharded_oracle(ty, m, exchange):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ty, m, exchange, q)) for r in range(2)]
    for p in procs:
        p.start()
    errs, same, argmax_ok = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    print(f"tp2 {exchange} ty={ty} m={m}: chained rel-L2 per seed {['%.1e' % e for e in errs]}")
    # (m > 1: wo, down and the head take f32 rows in the reference and two-level int8 rows here)
    assert np.median(errs) <= (1e-4 if m == 1 else 5e-4), errs
    assert sum(e > 2e-3 for e in errs) <= 1, errs
    assert same and argmax_ok


def _worker_causal(rank, world, port, ty, out_q):
    """The same two layers with the attention core: every rank keeps the f16 K/V rows of its own kv heads."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    from allpaka_b200 import gpu as G
    from allpaka_b200 import synth
    from oracle import oracle as orc
    from tests.test_gpu_attention import oracle_token
    from tests.util import Region, make_layer, oracle_logits, rel_l2, rope_table

    g = G.Gpu(rank)
    ids = [G.Gpu.dist_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    g.dist_init(rank, world, ids[0])
    handles = [None] * world
    dist.all_gather_object(handles, g.p2p_export())
    g.p2p_open(handles)
    hidden, nh, nkv, ffn, vocab, hd = 1024, 8, 2, 2048, 1536, 128
    d = dict(hidden=hidden, nq=nh * hd, nk=nkv * hd, hd=hd, ffn=ffn)
    layers = [make_layer(ty, hidden, d["nq"], d["nk"], ffn, 500 + 100 * l, True) for l in range(2)]
    head = synth.matrix(ty, vocab, hidden, 1999)
    names = ("wq", "wk", "wv", "wo", "gate", "up", "down")
    r = Region([L[n] for L in layers for n in names] + [head])
    assert g.attach(r.buf)
    tls = []
    for li, L in enumerate(layers):
        v = dict(zip(names, r.views[li * 7:(li + 1) * 7]))
        tls.append(G.TokenLayer(L["attn_norm"], L["ffn_norm"], (ty, v["wq"], d["nq"]), (ty, v["wk"], d["nk"]),
                                (ty, v["wv"], d["nk"]), (ty, v["wo"], hidden), (ty, v["gate"], ffn), (ty, v["up"], ffn),
                                (ty, v["down"], hidden), L["q_norm"], L["k_norm"]))
    out_norm = synth.gamma(hidden, 1998)
    cap = 16
    kv = G.KvCache(g, 2, d["nk"], cap)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    kcs = [np.zeros((cap, d["nk"]), np.uint16) for _ in range(2)]
    vcs = [np.zeros((cap, d["nk"]), np.uint16) for _ in range(2)]
    errs = []
    for pos in range(4):
        x = synth.normal_f32((1, hidden), 2100 + pos)
        rope = rope_table(orc, [pos], hd, hd)
        req = G.TokenReq(tls, out_norm, (ty, r.views[-1], vocab), x, 1, rope, hd, 1e-6, hidden, hd, nh, nkv,
                         attn_core=G.ATTN_CAUSAL, kv=kv, pos=pos, scale=scale)
        logits = g.decode_token_checked(req)
        if rank == 0:
            xo = oracle_token(orc, ty, layers, d, rope, x, 1, kcs, vcs, pos, scale)
            errs.append(rel_l2(logits, oracle_logits(orc, ty, head, vocab, hidden, xo, out_norm, 1e-6, 1)))
    if rank == 0:
        out_q.put(errs)
    dist.barrier()
    kv.close()
    g.close()
    dist.destroy_process_group()


def test_two_gpu_decode_with_the_attention_core():
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_causal, args=(r, 2, port, 8, q)) for r in range(2)]
    for p in procs:
        p.start()
    errs = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    print(f"tp2 with the attention core: logits rel-L2 per position {['%.1e' % e for e in errs]}")
    assert np.median(errs) <= 1e-4 and max(errs) <= 2e-2, errs

"""Tensor-parallel sharding on CPU: two gloo ranks slice the host tensors with the
library's own shard plan (apk_shard_plan, pure host arithmetic), compute their
shards with the CPU oracle, combine with all-reduce / all-gather, and must
reproduce the unsharded oracle.  Also: Q8 blocks of a K-slice are the same blocks,
so per-rank int32 block dots are the unsharded ones."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from allpaka_b200 import build, gpu, synth

Q8_0, Q4_K, Q5_K, Q6_K, Q5_0, Q3_K, Q2_K = 8, 12, 13, 14, 6, 11, 10


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rows(w, ty, n_out, n_in, r0, nr):
    rb = synth.expected_bytes(ty, n_in)
    return w.reshape(n_out, rb)[r0:r0 + nr].reshape(-1)


def _cols(w, ty, n_out, n_in, k0, nk):
    be, bb = synth.BLOCK[ty]
    rb = synth.expected_bytes(ty, n_in)
    return np.ascontiguousarray(w.reshape(n_out, rb)[:, k0 // be * bb:(k0 + nk) // be * bb]).reshape(-1)


def _worker(rank, world, port, ty, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as orc

    hidden, nh, nkv, hd, ffn, vocab = 512, 4, 2, 128, 1024, 768
    nq, nk = nh * hd, nkv * hd
    L = {n: synth.matrix(ty, o, i, 70 + j) for j, (n, o, i) in enumerate(
        [("wq", nq, hidden), ("wk", nk, hidden), ("wv", nk, hidden), ("wo", hidden, nq),
         ("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn), ("head", vocab, hidden)])}
    gam = synth.gamma(hidden, 80)
    x = synth.normal_f32(hidden, 81)
    inv = orc.rope_inv_freq(hd, 1e6)
    rope = orc.rope_sin_cos(4321, inv)[None]

    # ---- unsharded reference (every rank computes it; cheap at this size)
    q, k, v = orc.attn_in(ty, L["wq"], L["wk"], L["wv"], hidden, nq, nk, hd, x, 1, gam, 1e-6, rope)
    y_attn = orc.matmul(ty, L["wo"], hidden, nq, q, 1)[0]
    x1 = x + y_attn
    h = orc.rmsnorm_into(x1, gam, 1e-6)
    y_ffn, act = orc.ffn(ty, L["gate"], ty, L["up"], ty, L["down"], hidden, ffn, h, 1, return_act=True)
    logits = orc.matmul(ty, L["head"], vocab, hidden, h, 1)[0]

    # ---- this rank's shards, by the library's plan
    sq = gpu.shard_plan(gpu.SHARD_ROWS, ty, nq, hidden, rank, world, 128)
    sk = gpu.shard_plan(gpu.SHARD_ROWS, ty, nk, hidden, rank, world, 128)
    so = gpu.shard_plan(gpu.SHARD_K, ty, hidden, nq, rank, world)
    sf = gpu.shard_plan(gpu.SHARD_ROWS, ty, ffn, hidden, rank, world, 32)
    sd = gpu.shard_plan(gpu.SHARD_K, ty, hidden, ffn, rank, world)
    sh = gpu.shard_plan(gpu.SHARD_ROWS, ty, vocab, hidden, rank, world)
    assert sq[1] == so[3] and sq[0] == so[2], "a rank's Q heads are its wo columns"
    assert sf[1] == sd[3] and sf[0] == sd[2], "a rank's ffn rows are its down columns"

    ql, kl, vl = orc.attn_in(ty, _rows(L["wq"], ty, nq, hidden, sq[0], sq[1]), _rows(L["wk"], ty, nk, hidden, sk[0], sk[1]),
                             _rows(L["wv"], ty, nk, hidden, sk[0], sk[1]), hidden, sq[1], sk[1], hd, x, 1, gam, 1e-6, rope)
    assert np.array_equal(ql[0], q[0, sq[0]:sq[0] + sq[1]])  # column-parallel rows are bit-identical
    assert np.array_equal(kl[0], k[0, sk[0]:sk[0] + sk[1]])
    part = orc.matmul(ty, _cols(L["wo"], ty, hidden, nq, so[2], so[3]), hidden, so[3], ql, 1)[0]
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)  # the exchange after the row-parallel projection
    got_attn = t.numpy()

    # block dots of a K-slice are the unsharded ones
    _, _, qq = orc.q8acts(q[0])
    full_dots = orc.block_dots(ty, L["wo"], hidden, nq, qq)
    _, _, ql8 = orc.q8acts(ql[0])
    my_dots = orc.block_dots(ty, _cols(L["wo"], ty, hidden, nq, so[2], so[3]), hidden, so[3], ql8)
    assert np.array_equal(my_dots[0], full_dots[0][:, so[2] // 32:(so[2] + so[3]) // 32])

    g_l = orc.matmul(ty, _rows(L["gate"], ty, ffn, hidden, sf[0], sf[1]), sf[1], hidden, h, 1, orc.ACT_Q8)
    u_l = orc.matmul(ty, _rows(L["up"], ty, ffn, hidden, sf[0], sf[1]), sf[1], hidden, h, 1, orc.ACT_Q8)
    a_l = orc.swiglu(g_l, u_l)
    assert np.array_equal(a_l, act[0, sf[0]:sf[0] + sf[1]])
    part = orc.matmul(ty, _cols(L["down"], ty, hidden, ffn, sd[2], sd[3]), hidden, sd[3], a_l, 1)[0]
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    got_ffn = t.numpy()

    lg_l = orc.matmul(ty, _rows(L["head"], ty, vocab, hidden, sh[0], sh[1]), sh[1], hidden, h, 1)[0]
    parts = [torch.empty(sh[1]) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(lg_l.copy()))
    got_logits = torch.cat(parts).numpy()

    def rel(a, b):
        return float(np.linalg.norm(a.astype(np.float64) - b) / np.linalg.norm(b))

    res = (rel(got_attn, y_attn), rel(got_ffn, y_ffn[0]), bool(np.array_equal(got_logits, logits)))
    if rank == 0:
        out_q.put(res)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("ty", [Q8_0, Q5_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K])
def test_two_rank_tensor_parallel_layer_matches_unsharded_oracle(ty):
    build.build()
    from oracle import oracle

    oracle.build()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ty, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    e_attn, e_ffn, logits_equal = res
    # only the f32 summation order across ranks differs from the single-device result
    assert e_attn < 1e-5 and e_ffn < 1e-5
    assert logits_equal


def test_shard_plan_edges():
    build.build()
    assert gpu.shard_plan(gpu.SHARD_ROWS, Q8_0, 8192, 5120, 7, 8, 128) == (7168, 1024, 0, 5120)
    assert gpu.shard_plan(gpu.SHARD_K, Q8_0, 5120, 25600, 3, 8) == (0, 5120, 9600, 3200)
    assert gpu.shard_plan(gpu.SHARD_K, Q5_0, 5120, 25600, 3, 8) == (0, 5120, 9600, 3200)
    assert gpu.shard_plan(gpu.SHARD_K, Q4_K, 5120, 25600, 0, 8) is None      # 3200 is not whole super-blocks
    assert gpu.shard_plan(gpu.SHARD_K, Q4_K, 5120, 25600, 1, 4) == (0, 5120, 6400, 6400)
    assert gpu.shard_plan(gpu.SHARD_K, Q6_K, 5120, 25600, 0, 8) is None and gpu.shard_plan(gpu.SHARD_K, Q5_K, 5120, 25600, 0, 8) is None
    assert gpu.shard_plan(gpu.SHARD_K, Q6_K, 5120, 25600, 3, 4) == (0, 5120, 19200, 6400)
    assert gpu.shard_plan(gpu.SHARD_ROWS, Q8_0, 1024, 5120, 0, 16, 128) is None  # 8 kv heads over 16 ranks
    assert gpu.shard_plan(gpu.SHARD_ROWS, Q8_0, 151936, 5120, 1, 8) == (18992, 18992, 0, 5120)
    assert gpu.shard_plan(gpu.SHARD_ROWS, Q8_0, 100, 64, 0, 1) == (0, 100, 0, 64)

"""Committed golden fixtures (tests/golden/*.npz, made by tests/golden/make_golden.py).

CPU: the oracle still reproduces them bit for bit.  GPU: the CUDA path, through the
C ABI, matches them (int32 block dots and Q8 blocks exactly, f32 within 2e-3 rel-L2)."""
import os

import numpy as np
import pytest

from allpaka_b200 import synth
from tests.golden import make_golden
from tests.util import Region, make_layer, rel_l2, rope_table

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
Q8_0, Q4_K = 8, 12


def load(name):
    return dict(np.load(os.path.join(HERE, name + ".npz")))


@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_oracle_reproduces_the_golden_fixtures(orc, name):
    want = load(name)
    got = make_golden.CASES[name]()
    assert sorted(got) == sorted(want)
    for k in want:
        assert np.array_equal(np.asarray(got[k]), want[k]), (name, k)


@pytest.fixture(scope="module")
def gpu():
    from allpaka_b200 import gpu as G

    g = G.Gpu(0)
    yield g
    g.close()


@pytest.mark.gpu
def test_gpu_config0_against_golden(gpu):
    gold = load("config0")
    w = synth.q8_0_matrix(3072, 1024, 1000)
    x = synth.normal_f32(1024, 1001)
    r = Region([w])
    assert gpu.attach(r.buf)
    d, s, q = gpu.debug_q8_acts(x)
    assert np.array_equal(q, gold["q"]) and np.array_equal(d, gold["d"])
    dots = gpu.debug_block_dots(Q8_0, r.views[0], 1024, 3072, x, 1)
    assert np.array_equal(dots[0].sum(axis=1).astype(np.int64), gold["dots_rowsum"])
    assert np.array_equal(dots[0, :8], gold["dots_head"])
    assert rel_l2(gpu.matvec(Q8_0, r.views[0], 1024, 3072, x, 1)[0], gold["y"]) <= 1e-5
    gpu.detach(r.buf)


@pytest.mark.gpu
def test_gpu_q4k_against_golden(gpu):
    gold = load("q4k_small")
    w = synth.q4_k_matrix(384, 2048, 1100)
    x = synth.normal_f32((3, 2048), 1101)
    r = Region([w])
    assert gpu.attach(r.buf)
    dots = gpu.debug_block_dots(Q4_K, r.views[0], 2048, 384, x[0], 1)
    assert np.array_equal(dots[0].sum(axis=1).astype(np.int64), gold["dots_rowsum"])
    assert rel_l2(gpu.matvec(Q4_K, r.views[0], 2048, 384, x[0], 1)[0], gold["y1"]) <= 1e-5
    assert rel_l2(gpu.matvec(Q4_K, r.views[0], 2048, 384, x, 3, 0), gold["y3_q8"]) <= 1e-5
    assert rel_l2(gpu.matvec(Q4_K, r.views[0], 2048, 384, x, 3, 1), gold["y3_f32"]) <= 2e-3
    gpu.detach(r.buf)


@pytest.mark.gpu
def test_gpu_fused_paths_against_golden(gpu, orc):
    from allpaka_b200.gpu import FfnReq, TokenLayer, TokenReq

    gold = load("attn_small")
    hidden, nq, nk = 1024, 512, 256
    ws = [synth.q8_0_matrix(n, hidden, 1200 + i) for i, n in enumerate((nq, nk, nk))]
    r = Region(ws)
    assert gpu.attach(r.buf)
    _, x = synth.normal_bf16((2, hidden), 1203)
    rope = rope_table(orc, [31000, 7], 128, 128)
    q, k, v = gpu.attn_in(Q8_0, r.views[0], r.views[1], r.views[2], hidden, 128, 4, 2, x, 2, synth.gamma(hidden, 1204),
                          1e-6, rope, 128, synth.gamma(128, 1205), synth.gamma(128, 1206))
    for got, name in ((q, "q"), (k, "k"), (v, "v")):
        assert rel_l2(got, gold[name]) <= 2e-5, name
    gpu.detach(r.buf)

    gold = load("ffn_small")
    hidden, ffn = 1024, 2048
    ws = [synth.q8_0_matrix(ffn, hidden, 1300), synth.q8_0_matrix(ffn, hidden, 1301), synth.q8_0_matrix(hidden, ffn, 1302)]
    r = Region(ws)
    assert gpu.attach(r.buf)
    _, x = synth.normal_bf16((6, hidden), 1303)
    y1 = gpu.ffn_batch([FfnReq(Q8_0, r.views[0], Q8_0, r.views[1], Q8_0, r.views[2], hidden, ffn, x[0], 1)])[0]
    y6 = gpu.ffn_batch([FfnReq(Q8_0, r.views[0], Q8_0, r.views[1], Q8_0, r.views[2], hidden, ffn, x, 6)])[0]
    assert rel_l2(y1, gold["y1"]) <= 2e-5 and rel_l2(y6, gold["y6"]) <= 2e-3
    gpu.detach(r.buf)

    gold = load("token_small")
    hidden, nh, nkv, ffn, vocab = 512, 4, 2, 1024, 640
    layers = [make_layer(Q8_0, hidden, nh * 128, nkv * 128, ffn, 1400 + 100 * l, True) for l in range(2)]
    head = synth.q8_0_matrix(vocab, hidden, 1490)
    names = ("wq", "wk", "wv", "wo", "gate", "up", "down")
    r = Region([L[n] for L in layers for n in names] + [head])
    assert gpu.attach(r.buf)
    tls = []
    for li, L in enumerate(layers):
        vv = dict(zip(names, r.views[li * 7:(li + 1) * 7]))
        tls.append(TokenLayer(L["attn_norm"], L["ffn_norm"], (Q8_0, vv["wq"], nh * 128), (Q8_0, vv["wk"], nkv * 128),
                              (Q8_0, vv["wv"], nkv * 128), (Q8_0, vv["wo"], hidden), (Q8_0, vv["gate"], ffn),
                              (Q8_0, vv["up"], ffn), (Q8_0, vv["down"], hidden), L["q_norm"], L["k_norm"]))
    req = TokenReq(tls, synth.gamma(hidden, 1491), (Q8_0, r.views[-1], vocab), synth.normal_f32((1, hidden), 1492), 1,
                   rope_table(orc, [12345], 128, 128), 128, 1e-6, hidden, 128, nh, nkv)
    assert rel_l2(gpu.decode_token_checked(req), gold["logits"]) <= 2e-3
    gpu.detach(r.buf)

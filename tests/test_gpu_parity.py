"""CUDA path vs the CPU oracle, through the C ABI (run with -m gpu on a B200).

Bars: activation quantisation and int32 block dots bit-exact; every f32 output
within 2e-3 relative L2 of the oracle on identical seeded inputs.
"""
import numpy as np
import pytest

from allpaka_b200 import synth
from tests.util import (Q2_K, Q3_K, Q4_K, Q5_0, Q5_K, Q6_K, Q8_0, Region, make_layer, oracle_decode, oracle_logits, rel_l2,
                        rope_table)

pytestmark = pytest.mark.gpu

TOL = 2e-3  # relative L2 against the oracle


@pytest.fixture(scope="module")
def gpu():
    from allpaka_b200 import gpu as G

    g = G.Gpu(0)
    yield g
    g.close()


def attach(gpu, *parts):
    r = Region(parts)
    assert gpu.attach(r.buf)
    return r


# ---------------------------------------------------------------- activations

@pytest.mark.parametrize("n", [32, 256, 1024, 5120, 25600])
def test_q8_activation_blocks_are_bit_exact(gpu, orc, n):
    x = synth.normal_f32(n, 100 + n)
    x[: min(n, 64)] *= 1e-3
    if n >= 256:
        x[32:64] = 0.0  # an all-zero block: d = 0, q = 0
    d, s, q = gpu.debug_q8_acts(x)
    od, os_, oq = orc.q8acts(x)
    assert np.array_equal(q, oq)
    assert np.array_equal(d.view(np.uint32), od.view(np.uint32))
    assert np.array_equal(s.view(np.uint32), os_.view(np.uint32))


def test_rmsnorm_prologue_feeds_identical_blocks(gpu, orc):
    for seed, n in ((1, 5120), (2, 1024), (3, 256)):
        x = synth.normal_f32(n, seed) * 3.0
        g = synth.gamma(n, seed + 50)
        d, s, q = gpu.debug_q8_acts(x, gamma=g, eps=1e-6)
        h = orc.rmsnorm_into(x, g, 1e-6)
        od, os_, oq = orc.q8acts(h)
        assert np.array_equal(q, oq)
        assert np.array_equal(d.view(np.uint32), od.view(np.uint32))
        assert np.array_equal(s.view(np.uint32), os_.view(np.uint32))


# ------------------------------------------------------------------ block dots

@pytest.mark.parametrize("ty,n_out,n_in,m", [
    (Q8_0, 3072, 1024, 1),     # config 0
    (Q8_0, 130, 2048, 3),
    (Q8_0, 17, 64, 8),
    (Q4_K, 256, 1024, 1),
    (Q4_K, 200, 5120, 2),
    (Q4_K, 64, 256, 8),
    (Q5_K, 256, 1024, 1),
    (Q5_K, 200, 5120, 2),
    (Q5_K, 64, 256, 8),
    (Q6_K, 256, 1024, 1),     # per block: sc0*dot0 + sc1*dot1 of its two 16-element halves
    (Q6_K, 200, 5120, 2),
    (Q6_K, 130, 768, 4),
    (Q6_K, 64, 256, 8),
    (Q5_0, 3072, 1024, 1),    # q - 16 rebuilt from nibbles and the inverted fifth bits
    (Q5_0, 130, 2048, 3),
    (Q5_0, 200, 5120, 2),
    (Q5_0, 17, 64, 8),
    (Q5_0, 64, 288, 6),       # a last K-step of one block
    (Q3_K, 256, 1024, 1),     # carried in the Q6_K stream: sc0*dot0 + sc1*dot1 with the 3-bit values
    (Q3_K, 200, 5120, 2),
    (Q3_K, 64, 256, 8),
    (Q2_K, 256, 1024, 1),     # the scale-weighted part sc0*dot0 + sc1*dot1; the min term rides on the code sums
    (Q2_K, 200, 5120, 2),
    (Q2_K, 130, 768, 4),
    (Q2_K, 64, 256, 8),
])
def test_int32_block_dots_are_bit_exact(gpu, orc, ty, n_out, n_in, m):
    w = synth.matrix(ty, n_out, n_in, 7)
    r = attach(gpu, w)
    x = synth.normal_f32((m, n_in), 8)
    dots = gpu.debug_block_dots(ty, r.views[0], n_in, n_out, x, m)
    _, _, q = orc.q8acts(x)
    want = orc.block_dots(ty, w, n_out, n_in, q, m)
    assert np.array_equal(dots, want)
    gpu.detach(r.buf)


# --------------------------------------------------------------------- matvec

@pytest.mark.parametrize("n_out,n_in", [(1, 256), (48, 1024), (130, 768), (513, 5120), (64, 25600), (5120, 5120)])
@pytest.mark.parametrize("m", [1, 3, 4, 6, 8])
def test_q5_k_matvec_matches_oracle(gpu, orc, n_out, n_in, m):
    """dot_q5_k_i8 (q8_acts.rs:223-262) for Q8 activations, dot_q5_k (dot_f32.rs:97-135) for f32 ones."""
    w = synth.q5_k_matrix(n_out, n_in, 41)
    r = attach(gpu, w)
    x = synth.normal_f32((m, n_in), 42 + m)
    errs = []
    for mode, omode in ((0, orc.ACT_Q8), (1, orc.ACT_F32), (2, orc.ACT_AUTO)):
        got = gpu.matvec(Q5_K, r.views[0], n_in, n_out, x, m, mode)
        want = orc.matmul(Q5_K, w, n_out, n_in, x, m, omode)
        errs.append(rel_l2(got, want))
        assert errs[-1] <= TOL, (mode, errs)
        if mode == 0:
            assert errs[-1] <= 1e-5
    print(f"Q5_K {n_out}x{n_in} m={m}: rel-L2 q8 {errs[0]:.1e} f32 {errs[1]:.1e}")
    gpu.detach(r.buf)


@pytest.mark.parametrize("n_out,n_in", [(1, 256), (48, 1024), (130, 768), (513, 5120), (64, 25600), (5120, 5120)])
@pytest.mark.parametrize("m", [1, 3, 4, 6, 8])
def test_q2_k_matvec_matches_oracle(gpu, orc, n_out, n_in, m):
    """dot_q2_k_i8 (q8_acts.rs:127-174) for Q8 activations, dot_q2_k (dot_f32.rs:214-248) for f32 ones."""
    w = synth.q2_k_matrix(n_out, n_in, 71)
    r = attach(gpu, w)
    x = synth.normal_f32((m, n_in), 72 + m)
    errs = []
    for mode, omode in ((0, orc.ACT_Q8), (1, orc.ACT_F32), (2, orc.ACT_AUTO)):
        got = gpu.matvec(Q2_K, r.views[0], n_in, n_out, x, m, mode)
        want = orc.matmul(Q2_K, w, n_out, n_in, x, m, omode)
        errs.append(rel_l2(got, want))
        assert errs[-1] <= TOL, (mode, errs)
        if mode == 0:
            assert errs[-1] <= 1e-5  # integer dots and sums are exact; only the f32 accumulation order differs
    print(f"Q2_K {n_out}x{n_in} m={m}: rel-L2 q8 {errs[0]:.1e} f32 {errs[1]:.1e}")
    gpu.detach(r.buf)


@pytest.mark.parametrize("n_out,n_in", [(1, 256), (130, 768), (513, 5120), (64, 25600), (5120, 5120)])
@pytest.mark.parametrize("m", [1, 3, 6, 8])
def test_q3_k_matvec_matches_oracle(gpu, orc, n_out, n_in, m):
    """dot_q3_k_i8 (q8_acts.rs:178-218) for Q8 activations, dot_q3_k (dot_f32.rs:58-94) for f32 ones."""
    w = synth.q3_k_matrix(n_out, n_in, 61)
    r = attach(gpu, w)
    x = synth.normal_f32((m, n_in), 62 + m)
    errs = []
    for mode, omode in ((0, orc.ACT_Q8), (1, orc.ACT_F32), (2, orc.ACT_AUTO)):
        got = gpu.matvec(Q3_K, r.views[0], n_in, n_out, x, m, mode)
        want = orc.matmul(Q3_K, w, n_out, n_in, x, m, omode)
        errs.append(rel_l2(got, want))
        assert errs[-1] <= TOL, (mode, errs)
        if mode == 0:
            assert errs[-1] <= 1e-5  # integer dots are exact; only the f32 accumulation order differs
    print(f"Q3_K {n_out}x{n_in} m={m}: rel-L2 q8 {errs[0]:.1e} f32 {errs[1]:.1e}")
    gpu.detach(r.buf)


@pytest.mark.parametrize("n_out,n_in", [(1, 32), (48, 1024), (130, 800), (513, 5120), (64, 25600), (5120, 5120)])
@pytest.mark.parametrize("m", [1, 3, 4, 6, 8])
def test_q5_0_matvec_matches_oracle(gpu, orc, n_out, n_in, m):
    """dot_q5_0_i8 (q8_acts.rs:100-124) for Q8 activations, dot_q5_0 (dot_f32.rs:39-55) for f32 ones."""
    w = synth.q5_0_matrix(n_out, n_in, 51)
    r = attach(gpu, w)
    x = synth.normal_f32((m, n_in), 52 + m)
    errs = []
    for mode, omode in ((0, orc.ACT_Q8), (1, orc.ACT_F32), (2, orc.ACT_AUTO)):
        got = gpu.matvec(Q5_0, r.views[0], n_in, n_out, x, m, mode)
        want = orc.matmul(Q5_0, w, n_out, n_in, x, m, omode)
        errs.append(rel_l2(got, want))
        assert errs[-1] <= TOL, (mode, errs)
        if mode == 0:
            assert errs[-1] <= 1e-5  # integer dots are exact; only the f32 accumulation order differs
    print(f"Q5_0 {n_out}x{n_in} m={m}: rel-L2 q8 {errs[0]:.1e} f32 {errs[1]:.1e}")
    gpu.detach(r.buf)


@pytest.mark.parametrize("n_out,n_in", [(1, 256), (48, 1024), (130, 768), (513, 5120), (64, 25600), (5120, 5120)])
@pytest.mark.parametrize("m", [1, 3, 4, 6, 8])
def test_q6_k_matvec_matches_oracle(gpu, orc, n_out, n_in, m):
    """dot_q6_k_i8 (q8_acts.rs:307-346) for Q8 activations, dot_q6_k (dot_f32.rs:252-289) for f32 ones."""
    w = synth.q6_k_matrix(n_out, n_in, 31)
    r = attach(gpu, w)
    x = synth.normal_f32((m, n_in), 32 + m)
    errs = []
    for mode, omode in ((0, orc.ACT_Q8), (1, orc.ACT_F32), (2, orc.ACT_AUTO)):
        got = gpu.matvec(Q6_K, r.views[0], n_in, n_out, x, m, mode)
        want = orc.matmul(Q6_K, w, n_out, n_in, x, m, omode)
        errs.append(rel_l2(got, want))
        assert errs[-1] <= TOL, (mode, errs)
        if mode == 0:
            assert errs[-1] <= 1e-5  # integer dots are exact; only the f32 accumulation order differs
    print(f"Q6_K {n_out}x{n_in} m={m}: rel-L2 q8 {errs[0]:.1e} f32 {errs[1]:.1e}")
    gpu.detach(r.buf)


SHAPES = [(1, 32), (2, 64), (5, 256), (17, 512), (127, 1024), (128, 1024), (129, 288), (3072, 1024),
          (300, 5120), (64, 25600)]


@pytest.mark.parametrize("n_out,n_in", SHAPES)
@pytest.mark.parametrize("m", [1, 2, 5, 8])
def test_q8_0_matvec_matches_oracle(gpu, orc, n_out, n_in, m):
    w = synth.q8_0_matrix(n_out, n_in, 11)
    r = attach(gpu, w)
    x = synth.normal_f32((m, n_in), 12 + m)
    for mode, omode in ((0, orc.ACT_Q8), (1, orc.ACT_F32), (2, orc.ACT_AUTO)):
        got = gpu.matvec(Q8_0, r.views[0], n_in, n_out, x, m, mode)
        want = orc.matmul(Q8_0, w, n_out, n_in, x, m, omode)
        assert rel_l2(got, want) <= TOL, (mode, rel_l2(got, want))
        if mode == 0:
            assert rel_l2(got, want) <= 1e-5
    gpu.detach(r.buf)


@pytest.mark.parametrize("n_out,n_in", [(1, 256), (48, 1024), (130, 768), (513, 5120), (64, 25600)])
@pytest.mark.parametrize("m", [1, 3, 8])
def test_q4_k_matvec_matches_oracle(gpu, orc, n_out, n_in, m):
    w = synth.q4_k_matrix(n_out, n_in, 21)
    r = attach(gpu, w)
    x = synth.normal_f32((m, n_in), 22 + m)
    for mode, omode in ((0, orc.ACT_Q8), (1, orc.ACT_F32)):
        got = gpu.matvec(Q4_K, r.views[0], n_in, n_out, x, m, mode)
        want = orc.matmul(Q4_K, w, n_out, n_in, x, m, omode)
        assert rel_l2(got, want) <= TOL, (mode, rel_l2(got, want))
    gpu.detach(r.buf)


def test_config1_q4_k_ffn_gate_shape(gpu, orc):
    """Q4_K 25600x5120, batch 1."""
    n_out, n_in = 25600, 5120
    w = synth.q4_k_matrix(n_out, n_in, 1001)
    r = attach(gpu, w)
    x = synth.normal_f32(n_in, 1001 + 1)
    got = gpu.matvec(Q4_K, r.views[0], n_in, n_out, x, 1)
    want = orc.matmul(Q4_K, w, n_out, n_in, x, 1)
    assert rel_l2(got, want) <= 1e-5
    again = gpu.matvec(Q4_K, r.views[0], n_in, n_out, x, 1)
    assert np.array_equal(got, again)  # fixed summation order: run-to-run identical
    gpu.detach(r.buf)


def test_reference_cuda_parity_fixture(gpu, orc):
    """crates/allpaka-backend/tests/gpu_cuda_parity.rs:75-127: 8x64 Q8_0 out of an
    LCG-filled region, scales tamed, against dequant+dot with the reference's
    own tolerance (its kernel multiplies f32 activations, hence ACT_F32)."""
    region = synth.lcg_bytes(8 * 2 * 34, 0xC0FFEE00D15CAFE1)
    w = synth.tame_scales(region.copy(), Q8_0)
    r = attach(gpu, w)
    x = np.array([((i % 13) - 6.0) * 0.1 for i in range(64)], dtype=np.float32)
    got = gpu.matvec(Q8_0, r.views[0], 64, 8, x, 1, 1)[0]
    for j in range(8):
        row = orc.dequant(Q8_0, w[j * 68:(j + 1) * 68], 64)
        want = float(np.dot(row.astype(np.float64), x.astype(np.float64)))
        assert abs(got[j] - want) < 1e-3 + 1e-3 * abs(want)
    gpu.detach(r.buf)


def test_foreign_memory_and_bad_shapes_decline(gpu):
    """Weights outside every attached mapping decline (accel.rs:21-23); ragged rows and
    unknown types decline; nothing is computed on the CPU instead."""
    w = synth.q8_0_matrix(4, 64, 1)
    x = np.zeros(64, np.float32)
    assert gpu.matvec(Q8_0, w, 64, 4, x) is None
    assert gpu.last_decline[0] == 4
    r = attach(gpu, w)
    assert gpu.matvec(Q8_0, r.views[0], 64, 4, x) is not None
    assert gpu.matvec(99, r.views[0], 64, 4, x) is None and gpu.last_decline[0] == 2
    assert gpu.matvec(Q4_K, r.views[0], 64, 4, x) is None and gpu.last_decline[0] == 3
    assert gpu.matvec(Q8_0, r.views[0], 64, 4, np.zeros(9 * 64, np.float32), 9) is None
    gpu.detach(r.buf)
    assert gpu.matvec(Q8_0, r.views[0], 64, 4, x) is None  # detached: foreign again


def test_matvec_batch_shares_one_activation_quantisation(gpu, orc):
    from allpaka_b200.gpu import MatvecReq

    hidden = 1024
    ws = [synth.q8_0_matrix(n, hidden, 30 + i) for i, n in enumerate((512, 128, 128))]
    r = attach(gpu, *ws)
    x = synth.normal_f32((3, hidden), 33)
    reqs = [MatvecReq(Q8_0, v, hidden, n, x, 3) for v, n in zip(r.views, (512, 128, 128))]
    for v, n in zip(r.views, (512, 128, 128)):
        assert gpu.register_matrix(v, Q8_0, n, hidden)  # uploads happen here, not in the count below
    calls0 = gpu.stats()[1]
    ys = gpu.matvec_batch(reqs)
    assert gpu.stats()[1] - calls0 == 4  # one activation pass, three matvecs
    for y, w, n in zip(ys, ws, (512, 128, 128)):
        assert rel_l2(y, orc.matmul(Q8_0, w, n, hidden, x, 3, orc.ACT_Q8)) <= 1e-5
    gpu.detach(r.buf)


# ------------------------------------------------- fused prologue / epilogues

@pytest.mark.parametrize("m,qk_norm,rot_dim", [(1, False, 128), (1, True, 128), (3, True, 128), (2, False, 64)])
def test_config2_rmsnorm_qkv_rope(gpu, orc, m, qk_norm, rot_dim):
    """RMSNorm -> Q8_0 QKV 10240x5120 -> NeoX RoPE, Qwen3-32B attention shape, bf16 x."""
    hidden, hd, nh, nkv = 5120, 128, 64, 8
    nq, nk = nh * hd, nkv * hd
    wq = synth.q8_0_matrix(nq, hidden, 1002)
    wk = synth.q8_0_matrix(nk, hidden, 1003)
    wv = synth.q8_0_matrix(nk, hidden, 1004)
    r = attach(gpu, wq, wk, wv)
    _, x = synth.normal_bf16((m, hidden), 1005)
    gam = synth.gamma(hidden, 1006)
    qn = synth.gamma(hd, 1007) if qk_norm else None
    kn = synth.gamma(hd, 1008) if qk_norm else None
    pos = np.random.default_rng(1009).integers(0, 32768, size=m)
    rope = rope_table(orc, pos, hd, rot_dim)
    got = gpu.attn_in(Q8_0, r.views[0], r.views[1], r.views[2], hidden, hd, nh, nkv, x, m, gam, 1e-6, rope,
                      rot_dim, qn, kn)
    want = orc.attn_in(Q8_0, wq, wk, wv, hidden, nq, nk, hd, x, m, gam, 1e-6, rope, qn, kn)
    for g, w_, name in zip(got, want, "qkv"):
        assert rel_l2(g, w_) <= TOL, (name, rel_l2(g, w_))
        assert rel_l2(g, w_) <= 2e-5, (name, rel_l2(g, w_))
    gpu.detach(r.buf)


@pytest.mark.parametrize("m", [1, 6])
def test_config3_ffn_swiglu_down(gpu, orc, m):
    """gate, up 25600x5120 with fused SwiGLU, then down 5120x25600 (Q8_0), bf16 x."""
    from allpaka_b200.gpu import FfnReq

    hidden, ffn = 5120, 25600
    g = synth.q8_0_matrix(ffn, hidden, 1010)
    u = synth.q8_0_matrix(ffn, hidden, 1011)
    d = synth.q8_0_matrix(hidden, ffn, 1012)
    r = attach(gpu, g, u, d)
    _, x = synth.normal_bf16((m, hidden), 1013)
    got = gpu.ffn_batch([FfnReq(Q8_0, r.views[0], Q8_0, r.views[1], Q8_0, r.views[2], hidden, ffn, x, m)])[0]
    want = orc.ffn(Q8_0, g, Q8_0, u, Q8_0, d, hidden, ffn, x, m)
    err = rel_l2(got, want)
    print(f"config 3, m = {m}: rel-L2 {err:.2e}")
    # m = 1: `down` takes Q8 blocks of the SwiGLU row; expf differs in its last bit between libm and
    # the device, and of 25 600 values a few then round to the neighbouring code (measured 1.2e-4).
    # m = 6: `down` takes f32 rows in the reference and two-level int8 rows here (measured 3.5e-5).
    assert err <= (5e-4 if m == 1 else 1e-4), err
    gpu.detach(r.buf)


@pytest.mark.parametrize("ty,hidden,ffn,m", [(Q8_0, 256, 96, 1), (Q8_0, 512, 1024, 5), (Q4_K, 512, 1024, 1),
                                             (Q4_K, 512, 1024, 4)])
def test_small_ffn(gpu, orc, ty, hidden, ffn, m):
    from allpaka_b200.gpu import FfnReq

    if ty == Q4_K and ffn % 256:
        pytest.skip("Q4_K rows are whole 256-element super-blocks")
    g = synth.matrix(ty, ffn, hidden, 40)
    u = synth.matrix(ty, ffn, hidden, 41)
    d = synth.matrix(ty, hidden, ffn, 42)
    r = attach(gpu, g, u, d)
    x = synth.normal_f32((m, hidden), 43)
    got = gpu.ffn_batch([FfnReq(ty, r.views[0], ty, r.views[1], ty, r.views[2], hidden, ffn, x, m)])[0]
    want = orc.ffn(ty, g, ty, u, ty, d, hidden, ffn, x, m)
    assert rel_l2(got, want) <= TOL, rel_l2(got, want)
    gpu.detach(r.buf)


# ------------------------------------------------------------------ whole token

def build_token(gpu, orc, ty, n_layers, hidden, nh, nkv, ffn, vocab, m, qk_norm, seed):
    from allpaka_b200.gpu import TokenLayer, TokenReq

    hd = 128
    nq, nk = nh * hd, nkv * hd
    layers = [make_layer(ty, hidden, nq, nk, ffn, seed + 100 * l, qk_norm) for l in range(n_layers)]
    head = synth.matrix(ty, vocab, hidden, seed + 9000)
    names = ("wq", "wk", "wv", "wo", "gate", "up", "down")
    r = attach(gpu, *[L[n] for L in layers for n in names], head)
    tls = []
    for li, L in enumerate(layers):
        v = dict(zip(names, r.views[li * 7:(li + 1) * 7]))
        tls.append(TokenLayer(L["attn_norm"], L["ffn_norm"], (ty, v["wq"], nq), (ty, v["wk"], nk),
                              (ty, v["wv"], nk), (ty, v["wo"], hidden), (ty, v["gate"], ffn),
                              (ty, v["up"], ffn), (ty, v["down"], hidden), L.get("q_norm"), L.get("k_norm")))
    out_norm = synth.gamma(hidden, seed + 9001)
    x = synth.normal_f32((m, hidden), seed + 9002)
    pos = np.arange(m) + 1234
    rope = rope_table(orc, pos, hd, hd)
    req = TokenReq(tls, out_norm, (ty, r.views[-1], vocab), x, m, rope, hd, 1e-6, hidden, hd, nh, nkv)
    return req, layers, head, out_norm, x, rope, r


@pytest.mark.parametrize("ty,m,qk_norm", [(Q8_0, 1, False), (Q8_0, 1, True), (Q8_0, 4, True), (Q4_K, 1, False),
                                           (Q4_K, 3, True), (Q5_0, 1, True), (Q5_0, 3, False), (Q3_K, 1, True), (Q2_K, 1, True), (Q2_K, 3, False)])
def test_decode_token_matches_oracle_layer_stack(gpu, orc, ty, m, qk_norm):
    hidden, nh, nkv, ffn, vocab = 512, 4, 2, 1024, 1000
    req, layers, head, out_norm, x, rope, r = build_token(gpu, orc, ty, 3, hidden, nh, nkv, ffn, vocab, m, qk_norm, 500)
    logits = gpu.decode_token_checked(req)
    xo = oracle_decode(orc, ty, layers, hidden, nh * 128, nkv * 128, 128, ffn, 1e-6, rope, x, m)
    want = oracle_logits(orc, ty, head, vocab, hidden, xo, out_norm, 1e-6, m)
    assert rel_l2(logits, want) <= TOL, rel_l2(logits, want)
    again = gpu.decode_token_checked(req)
    assert np.array_equal(logits, again)
    req.argmax = True
    ids = gpu.decode_token_checked(req)
    ids = ids.argmax if m > 1 else ids  # a verify batch answers with TokenOut::Rows
    assert list(ids) == [int(np.flatnonzero(row == row.max())[-1]) for row in logits]
    st = gpu.decode_path_stats()
    assert st["successes"] >= 3 and st["attempts"] >= st["successes"]
    gpu.detach(r.buf)


@pytest.mark.parametrize("ty,m", [(Q8_0, 1), (Q8_0, 3), (Q4_K, 1), (Q5_K, 1), (Q6_K, 1)])
def test_decode_token_tiles_shared_by_many_ctas(gpu, orc, ty, m):
    """Shapes whose K dimension spreads one tile over up to eight CTAs (every CTA holds one unit),
    per-head norm on: the cross-CTA hand-off, the residual epilogue and the packed Q for wo."""
    hidden, nh, nkv, ffn, vocab = 1024, 8, 2, 2048, 1536
    req, layers, head, out_norm, x, rope, r = build_token(gpu, orc, ty, 2, hidden, nh, nkv, ffn, vocab, m, True, 700)
    logits = gpu.decode_token_checked(req)
    xo = oracle_decode(orc, ty, layers, hidden, nh * 128, nkv * 128, 128, ffn, 1e-6, rope, x, m)
    want = oracle_logits(orc, ty, head, vocab, hidden, xo, out_norm, 1e-6, m)
    assert rel_l2(logits, want) <= TOL, rel_l2(logits, want)
    assert np.array_equal(logits, gpu.decode_token_checked(req))
    gpu.detach(r.buf)


@pytest.mark.parametrize("ty,m", [(Q8_0, 1), (Q8_0, 5), (Q4_K, 2)])
def test_next_norm_started_by_the_residual_epilogue_changes_nothing(orc, ty, m, monkeypatch):
    """The RMSNorm in front of Q|K|V, gate/up and the head either adds up the per-block sums of squares
    that the residual epilogue left (default), reduces the row itself (0), or takes records that the
    residual epilogue already quantised before the row scale existed (2, opt-in approximation): same logits."""
    from allpaka_b200 import gpu as G

    out = []
    for fuse in ("1", "0", "2"):
        monkeypatch.setenv("ALLPAKA_B200_FUSE_NORM", fuse)
        g = G.Gpu(0)
        req, layers, head, out_norm, x, rope, r = build_token(g, orc, ty, 2, 1024, 8, 2, 2048, 1536, m, True, 800)
        out.append(g.decode_token_checked(req))
        if fuse == "1":
            xo = oracle_decode(orc, ty, layers, 1024, 8 * 128, 2 * 128, 128, 2048, 1e-6, rope, x, m)
            want = oracle_logits(orc, ty, head, 1536, 1024, xo, out_norm, 1e-6, m)
            assert rel_l2(out[0], want) <= TOL, rel_l2(out[0], want)
        g.detach(r.buf)
        g.close()
    assert rel_l2(out[0], out[1]) <= 1e-6, rel_l2(out[0], out[1])
    assert rel_l2(out[0], out[2]) <= 1e-3, rel_l2(out[0], out[2])


def test_token_timeline_is_ordered(gpu, orc):
    """Trace entry point: one slab of stamps per matvec launch, entry <= dependency <= last tile closed."""
    req, layers, head, out_norm, x, rope, r = build_token(gpu, orc, Q8_0, 2, 512, 4, 2, 1024, 1000, 1, False, 900)
    st = gpu.debug_token_timeline(req, 16).astype(np.int64)
    assert st.shape[0] == 2 * 4 + 1 and st.shape[2] == 8
    for slab in st:
        live = slab[(slab[:, 0] > 0) & (slab[:, 2] > 0)]  # CTAs that got work (a late one finds no chunk left and leaves at once)
        assert len(live) > 0
        assert np.all(live[:, 2] >= live[:, 0]) and np.all(live[:, 5] >= live[:, 2])
    ends = [slab[:, 5].max() for slab in st]
    assert all(b > a for a, b in zip(ends, ends[1:]))  # launches finish in issue order
    gpu.detach(r.buf)


def test_decode_token_declines_what_it_does_not_build(gpu, orc):
    from allpaka_b200.gpu import DecodeDecline

    req, *_rest, r = build_token(gpu, orc, Q8_0, 1, 512, 4, 2, 1024, 1000, 1, False, 700)
    req.attn_core = 0
    with pytest.raises(DecodeDecline):
        gpu.decode_token_checked(req)
    assert gpu.decode_token(req) is None
    req.attn_core = 1
    req.m = 9
    req.x = np.zeros((9, 512), np.float32)
    with pytest.raises(DecodeDecline):
        gpu.decode_token_checked(req)
    gpu.detach(r.buf)


def test_one_qwen3_32b_shaped_layer(gpu, orc):
    """One layer of the benchmark stack at full width (hidden 5120, 64+8 heads, ffn 25600)."""
    hidden, nh, nkv, ffn, vocab = 5120, 64, 8, 25600, 4096
    req, layers, head, out_norm, x, rope, r = build_token(gpu, orc, Q8_0, 1, hidden, nh, nkv, ffn, vocab, 1, False, 2000)
    logits = gpu.decode_token_checked(req)
    xo = oracle_decode(orc, Q8_0, layers, hidden, nh * 128, nkv * 128, 128, ffn, 1e-6, rope, x, 1)
    want = oracle_logits(orc, Q8_0, head, vocab, hidden, xo, out_norm, 1e-6, 1)
    assert rel_l2(logits, want) <= TOL, rel_l2(logits, want)
    ms = gpu.decode_replay(req, 3)
    assert ms > 0
    gpu.detach(r.buf)

"""Decode attention over the f16 KV cache, and the decoder layer with it in place of the
identity stand-in (model/attention.rs:337-428 attend_group / attend_one; model/kv.rs:682-697 the
f16 store; gpu/types.rs:34-52 AttnReq).  Floating point throughout: the bar is the 2e-3 relative
L2 of the path, the measured figures are at rounding level and asserted two decades tighter."""
import numpy as np
import pytest

from allpaka_b200 import synth
from tests.util import Q4_K, Q8_0, Region, make_layer, oracle_logits, rel_l2, rope_table

pytestmark = pytest.mark.gpu


def f16_rows(orc, rows):
    return np.stack([orc.kv_store(r) for r in rows])


@pytest.mark.parametrize("n_heads,n_kv,n_pos,m", [(8, 2, 33, 1), (64, 8, 700, 1), (16, 16, 257, 3), (8, 1, 1, 1),
                                                    (32, 4, 4096, 2), (32, 8, 300, 8), (8, 4, 150, 7),
                                                    (12, 1, 90, 3), (64, 8, 130, 5), (32, 8, 3, 8)])
def test_attention_core_matches_attend_one(orc, n_heads, n_kv, n_pos, m):
    from allpaka_b200 import gpu as G

    g = G.Gpu(0)
    hd, kv_dim, group = 128, n_kv * 128, n_heads // n_kv
    cap = n_pos + m + 5
    kv = G.KvCache(g, 2, kv_dim, cap)
    rng = np.random.default_rng(n_pos)
    k = f16_rows(orc, rng.standard_normal((n_pos + m - 1, kv_dim)).astype(np.float32))
    v = f16_rows(orc, rng.standard_normal((n_pos + m - 1, kv_dim)).astype(np.float32))
    kv.write(1, 0, k, v)
    rk, rv = kv.read(1, 0, n_pos + m - 1)
    assert np.array_equal(rk, k) and np.array_equal(rv, v)
    q = (rng.standard_normal((m, n_heads * hd)) * 2.0).astype(np.float32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    pos = n_pos - 1
    got = g.attend(kv, 1, q, m, n_heads, pos, scale)
    want = np.stack([orc.attend_one(q[i], k, v, kv_dim, n_kv, hd, group, 0, pos + i, scale) for i in range(m)])
    err = rel_l2(got, want)
    print(f"attention {n_heads}/{n_kv} heads, {n_pos} positions, m={m}: rel-L2 {err:.1e}")
    assert err <= 2e-5
    assert g.attend(kv, 1, q, m, n_heads, cap, scale) is None  # past the cache
    kv.close()
    g.close()


def test_attention_core_on_cuda_cores_agrees(orc, monkeypatch):
    """ALLPAKA_B200_ATTN_TC=0 selects the f32 CUDA-core form of the split kernel (the default feeds the tensor
    cores with hi + lo f16 fragments of q and of the softmax weights): both sit at rounding level of the oracle."""
    from allpaka_b200 import gpu as G

    outs = []
    for tc in ("1", "0"):
        monkeypatch.setenv("ALLPAKA_B200_ATTN_TC", tc)
        g = G.Gpu(0)
        n_heads, n_kv, n_pos, hd = 40, 8, 1500, 128
        kv = G.KvCache(g, 1, n_kv * hd, n_pos)
        rng = np.random.default_rng(77)
        k = f16_rows(orc, rng.standard_normal((n_pos, n_kv * hd)).astype(np.float32))
        v = f16_rows(orc, rng.standard_normal((n_pos, n_kv * hd)).astype(np.float32))
        kv.write(0, 0, k, v)
        q = (rng.standard_normal((2, n_heads * hd)) * 3.0).astype(np.float32)
        scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
        got = g.attend(kv, 0, q, 2, n_heads, n_pos - 2, scale)
        want = np.stack([orc.attend_one(q[i], k, v, n_kv * hd, n_kv, hd, n_heads // n_kv, 0, n_pos - 2 + i, scale) for i in range(2)])
        err = rel_l2(got, want)
        print(f"attention core, tensor cores {tc}: rel-L2 {err:.1e}")
        assert err <= 2e-5
        outs.append(got)
        kv.close()
        g.close()
    assert rel_l2(outs[0], outs[1]) <= 2e-5


def oracle_token(orc, ty, layers, d, rope, x, m, kcs, vcs, pos, scale):
    """The reference's layer order with the real attention core: K (roped) and V of the m rows go into
    the cache as f16 at pos..pos+m-1, row i attends over 0..=pos+i (model/decode.rs:435-591,
    model/attention.rs:78-330)."""
    hidden, nq, nk, hd, ffn = d["hidden"], d["nq"], d["nk"], d["hd"], d["ffn"]
    x = np.array(x, np.float32).reshape(m, hidden).copy()
    for li, L in enumerate(layers):
        q, k, v = orc.attn_in(ty, L["wq"], L["wk"], L["wv"], hidden, nq, nk, hd, x, m, L["attn_norm"], 1e-6, rope,
                              L.get("q_norm"), L.get("k_norm"))
        for i in range(m):
            kcs[li][pos + i], vcs[li][pos + i] = orc.kv_store(k[i]), orc.kv_store(v[i])
        att = np.stack([orc.attend_one(q[i], kcs[li], vcs[li], nk, nk // hd, hd, nq // nk, 0, pos + i, scale) for i in range(m)])
        x = x + orc.matmul(ty, L["wo"], hidden, nq, att, m)
        h = np.stack([orc.rmsnorm_into(x[i], L["ffn_norm"], 1e-6) for i in range(m)])
        x = x + orc.ffn(ty, L["gate"], ty, L["up"], ty, L["down"], hidden, ffn, h, m)
    return x


@pytest.mark.parametrize("ty,m", [(Q8_0, 1), (Q8_0, 3), (Q4_K, 1)])
def test_decoder_layers_with_the_attention_core(orc, ty, m):
    from allpaka_b200 import gpu as G

    g = G.Gpu(0)
    hidden, nh, nkv, ffn, vocab, hd = 512, 4, 2, 1024, 1000, 128
    d = dict(hidden=hidden, nq=nh * hd, nk=nkv * hd, hd=hd, ffn=ffn)
    layers = [make_layer(ty, hidden, d["nq"], d["nk"], ffn, 8100 + 100 * l, True) for l in range(2)]
    head = synth.matrix(ty, vocab, hidden, 8900)
    names = ("wq", "wk", "wv", "wo", "gate", "up", "down")
    r = Region([L[n] for L in layers for n in names] + [head])
    assert g.attach(r.buf)
    tls = []
    for li, L in enumerate(layers):
        v = dict(zip(names, r.views[li * 7:(li + 1) * 7]))
        tls.append(G.TokenLayer(L["attn_norm"], L["ffn_norm"], (ty, v["wq"], d["nq"]), (ty, v["wk"], d["nk"]),
                                (ty, v["wv"], d["nk"]), (ty, v["wo"], hidden), (ty, v["gate"], ffn), (ty, v["up"], ffn),
                                (ty, v["down"], hidden), L["q_norm"], L["k_norm"]))
    out_norm = synth.gamma(hidden, 8901)
    cap = 64
    kv = G.KvCache(g, 2, d["nk"], cap)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    kcs = [np.zeros((cap, d["nk"]), np.uint16) for _ in range(2)]
    vcs = [np.zeros((cap, d["nk"]), np.uint16) for _ in range(2)]
    pos = 0
    worst = 0.0
    for step in range(5):   # five consecutive calls grow the cache: each attends over everything before it
        x = synth.normal_f32((m, hidden), 8200 + step)
        rope = rope_table(orc, np.arange(m) + pos, hd, hd)
        req = G.TokenReq(tls, out_norm, (ty, r.views[-1], vocab), x, m, rope, hd, 1e-6, hidden, hd, nh, nkv,
                         attn_core=G.ATTN_CAUSAL, kv=kv, pos=pos, scale=scale)
        logits = g.decode_token_checked(req)
        xo = oracle_token(orc, ty, layers, d, rope, x, m, kcs, vcs, pos, scale)
        want = oracle_logits(orc, ty, head, vocab, hidden, xo, out_norm, 1e-6, m)
        worst = max(worst, rel_l2(logits, want))
        pos += m
    # the cache the GPU built holds the oracle's halves (K after per-head norm and RoPE, V as projected)
    for li in range(2):
        gk, gv = kv.read(li, 0, pos)
        fk = np.frombuffer(gk.tobytes(), np.float16).astype(np.float32)
        wk = np.frombuffer(kcs[li][:pos].tobytes(), np.float16).astype(np.float32)
        fv = np.frombuffer(gv.tobytes(), np.float16).astype(np.float32)
        wv = np.frombuffer(vcs[li][:pos].tobytes(), np.float16).astype(np.float32)
        assert rel_l2(fk, wk) <= 1e-3 and rel_l2(fv, wv) <= 1e-3
        if li == 0:  # layer 0 sees identical inputs: its rows differ from the oracle's by a half ulp at most, rarely
            assert np.mean(gk != kcs[0][:pos]) < 0.01 and np.mean(gv != vcs[0][:pos]) < 0.01
    print(f"decoder with attention, ty {ty} m={m}: worst logits rel-L2 over 5 calls {worst:.1e}")
    assert worst <= 2e-3
    req.pos = cap  # past capacity: declined, nothing written
    with pytest.raises(G.DecodeDecline):
        g.decode_token_checked(req)
    kv.close()
    g.detach(r.buf)
    g.close()


def test_greedy_chain_over_the_kv_cache(orc):
    """decode_greedy_continue with the attention core: each step stores its K/V rows at the next cache
    position (advanced on the device) and attends over everything before it.  The chain of n steps with
    one synchronisation gives the ids of n single argmax calls, and leaves the same cache."""
    from allpaka_b200 import gpu as G
    from tests.test_gpu_token_ends import build

    g = G.Gpu(0)
    req, layers, head, embd, out_norm, d, r = build(g, orc, Q8_0, True, 7700)
    n, pos0, tok0, cap = 6, 3, 41, 16
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d["hd"])))
    ropes = rope_table(orc, np.arange(n) + pos0, d["hd"], d["hd"])
    rng = np.random.default_rng(5)
    pre_k = f16_rows(orc, rng.standard_normal((pos0, d["nk"])).astype(np.float32))
    pre_v = f16_rows(orc, rng.standard_normal((pos0, d["nk"])).astype(np.float32))
    caches = []
    for _ in range(2):
        kv = G.KvCache(g, 2, d["nk"], cap)
        for layer in range(2):
            kv.write(layer, 0, pre_k, pre_v)   # a prefill handed over from elsewhere
        caches.append(kv)
    req.attn_core, req.scale = G.ATTN_CAUSAL, scale
    req.kv, req.pos, req.token_id = caches[0], pos0, tok0
    chain = g.decode_greedy(req, n, ropes)
    assert chain is not None
    tok, single = tok0, []
    req.kv, req.argmax = caches[1], True
    for i in range(n):
        req.token_id, req.rope, req.pos = tok, ropes[i:i + 1], pos0 + i
        tok = int(g.decode_token_checked(req)[0])
        single.append(tok)
    assert [int(t) for t in chain] == single
    for layer in range(2):
        ka, va = caches[0].read(layer, 0, pos0 + n)
        kb, vb = caches[1].read(layer, 0, pos0 + n)
        assert np.array_equal(ka, kb) and np.array_equal(va, vb)
        assert np.array_equal(ka[:pos0], pre_k)
    req.pos, req.kv = cap - 2, caches[0]
    assert g.decode_greedy(req, n, ropes) is None and g.last_decline[0] == 6   # would run past the cache
    for kv in caches:
        kv.close()
    g.detach(r.buf)
    g.close()

"""Token ends on the GPU: the input row from the embedding table by token id, the greedy winner,
and the greedy chain that feeds each winner back as the next input without returning to the host
(gpu/types.rs:187-192 `TokenReq.embd/token_id`; gpu/cuda/decode.rs:93-227 `decode_greedy_continue`;
model/decode.rs:422-431 `embed_token`, 604-608 greedy pick with ties to the higher id)."""
import numpy as np
import pytest

from allpaka_b200 import synth
from tests.util import Q2_K, Q3_K, Q4_K, Q5_0, Q5_K, Q6_K, Q8_0, Region, make_layer, oracle_decode, oracle_logits, rel_l2, rope_table

pytestmark = pytest.mark.gpu


def build(g, orc, ty, tied, seed):
    from allpaka_b200.gpu import TokenLayer, TokenReq

    hidden, nh, nkv, ffn, vocab, hd = 512, 4, 2, 1024, 1000, 128
    nq, nk = nh * hd, nkv * hd
    layers = [make_layer(ty, hidden, nq, nk, ffn, seed + 100 * l, True) for l in range(2)]
    head = synth.matrix(ty, vocab, hidden, seed + 9000)
    embd = head if tied else synth.matrix(ty, vocab, hidden, seed + 9500)
    names = ("wq", "wk", "wv", "wo", "gate", "up", "down")
    r = Region([L[n] for L in layers for n in names] + [head] + ([] if tied else [embd]))
    assert g.attach(r.buf)
    tls = []
    for li, L in enumerate(layers):
        v = dict(zip(names, r.views[li * 7:(li + 1) * 7]))
        tls.append(TokenLayer(L["attn_norm"], L["ffn_norm"], (ty, v["wq"], nq), (ty, v["wk"], nk), (ty, v["wv"], nk),
                              (ty, v["wo"], hidden), (ty, v["gate"], ffn), (ty, v["up"], ffn), (ty, v["down"], hidden),
                              L["q_norm"], L["k_norm"]))
    out_norm = synth.gamma(hidden, seed + 9001)
    head_v = r.views[14]
    embd_v = head_v if tied else r.views[15]
    req = TokenReq(tls, out_norm, (ty, head_v, vocab), None, 1, None, hd, 1e-6, hidden, hd, nh, nkv,
                   embd=(ty, embd_v, vocab))
    dims = dict(hidden=hidden, nq=nq, nk=nk, ffn=ffn, vocab=vocab, hd=hd)
    return req, layers, head, embd, out_norm, dims, r


def embed_row(orc, ty, embd, hidden, tok):
    rb = synth.expected_bytes(ty, hidden)
    return orc.dequant(ty, embd[tok * rb:(tok + 1) * rb], hidden)


@pytest.mark.parametrize("ty,tied", [(Q8_0, True), (Q8_0, False), (Q4_K, True), (Q5_K, True), (Q6_K, True), (Q5_0, True), (Q3_K, True), (Q2_K, True)])
def test_input_row_by_token_id(orc, ty, tied):
    from allpaka_b200 import gpu as G

    g = G.Gpu(0)
    req, layers, head, embd, out_norm, d, r = build(g, orc, ty, tied, 7100)
    for tok in (0, 1, 127, 128, 511, 999):
        req.x, req.token_id = None, tok
        req.rope = rope_table(orc, [40 + tok], d["hd"], d["hd"])
        by_id = g.decode_token_checked(req)
        x = embed_row(orc, ty, embd, d["hidden"], tok)
        req.x, req.token_id = x[None], None
        by_x = g.decode_token_checked(req)
        assert np.array_equal(by_id, by_x)  # the row dequantised on the device is the reference's row, bit for bit
        xo = oracle_decode(orc, ty, layers, d["hidden"], d["nq"], d["nk"], d["hd"], d["ffn"], 1e-6, req.rope, x, 1)
        want = oracle_logits(orc, ty, head, d["vocab"], d["hidden"], xo, out_norm, 1e-6, 1)
        assert rel_l2(by_id, want) <= 2e-3
    req.x, req.token_id = None, d["vocab"]
    with pytest.raises(Exception):
        g.decode_token_checked(req)  # out of vocabulary
    g.detach(r.buf)
    g.close()


@pytest.mark.parametrize("ty,tied", [(Q8_0, True), (Q4_K, False)])
def test_greedy_chain_follows_the_oracle(orc, ty, tied):
    from allpaka_b200 import gpu as G

    g = G.Gpu(0)
    req, layers, head, embd, out_norm, d, r = build(g, orc, ty, tied, 7300)
    n, pos0, tok0 = 8, 321, 17
    ropes = rope_table(orc, np.arange(n) + pos0, d["hd"], d["hd"])
    req.token_id = tok0
    got = g.decode_greedy(req, n, ropes)
    assert got is not None and got.shape == (n,)
    tok, want, margins = tok0, [], []
    for i in range(n):
        x = embed_row(orc, ty, embd, d["hidden"], tok)
        xo = oracle_decode(orc, ty, layers, d["hidden"], d["nq"], d["nk"], d["hd"], d["ffn"], 1e-6, ropes[i:i + 1], x, 1)
        lg = oracle_logits(orc, ty, head, d["vocab"], d["hidden"], xo, out_norm, 1e-6, 1)[0]
        tok = int(np.flatnonzero(lg == lg.max())[-1])
        top2 = np.sort(lg)[-2:]
        margins.append(float(top2[1] - top2[0]) / float(np.abs(lg).max()))
        want.append(tok)
    print(f"greedy chain: {list(got)} vs oracle {want}; smallest winner margin {min(margins):.1e} of the largest logit")
    assert [int(t) for t in got] == want
    # the same chain step by step through decode_token (argmax) gives the same ids
    tok, single = tok0, []
    req.argmax = True
    for i in range(n):
        req.token_id, req.rope = tok, ropes[i:i + 1]
        tok = int(g.decode_token_checked(req)[0])
        single.append(tok)
    assert single == want
    st = g.decode_path_stats()
    assert st["successes"] >= 2 * n
    g.detach(r.buf)
    g.close()

"""A model file end to end: GGUF written here -> reader -> model view -> attach -> tokens by id
through the decode path with the attention core and the f16 KV cache, against the oracle's
restatement of the same layer order on the file's own tensors."""
import numpy as np
import pytest

from allpaka_b200 import gguf
from tests.test_gguf_reader import tiny_model
from tests.util import Q2_K, Q3_K, Q4_K, Q5_0, Q5_K, Q6_K, Q8_0, oracle_logits, rel_l2, rope_table

pytestmark = pytest.mark.gpu


def rope_norm_rows(x, table, head_dim):
    """rope_norm_cached_from_array (ops/rope.rs:52-67) on every head of a row: pairs (2i, 2i+1)."""
    x = x.reshape(-1, head_dim).copy()
    for i, (sin, cos) in enumerate(table):
        a, b = x[:, 2 * i].copy(), x[:, 2 * i + 1].copy()
        x[:, 2 * i] = a * cos - b * sin
        x[:, 2 * i + 1] = a * sin + b * cos
    return x.reshape(-1)


def oracle_step(orc, f, info, x, pos, kcs, vcs, pairwise):
    """One token through the file's layers, every matrix in the type the file gives it
    (model/decode.rs:435-591 with model/attention.rs:78-330: per-head norm, then the rotation)."""
    H, hd, nh, nkv = info["hidden"], info["head_dim"], info["n_heads"], info["n_kv_heads"]
    nq, nk, ffn, eps = nh * hd, nkv * hd, info["ffn"], info["eps"]
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    inv = orc.rope_inv_freq(info["rot_dim"], info["rope_base"])
    table = orc.rope_sin_cos(pos, inv)

    def mm(name, n_out, n_in, rows):
        t = f.tensor(name)
        return orc.matmul(t["ty"], t["data"], n_out, n_in, rows, 1)

    def v32(name):
        t = f.tensor(name)
        return None if t is None else t["data"].view(np.float32)

    def heads(row, norm):
        out = row.reshape(-1, hd).copy()
        for i in range(out.shape[0]):
            if norm is not None:
                out[i] = orc.rmsnorm(out[i], norm, eps)
            out[i] = rope_norm_rows(out[i], table, hd) if pairwise else orc.rope_neox_table(out[i], table)
        return out.reshape(-1)

    x = np.array(x, np.float32).reshape(1, H)
    for l in range(info["n_layers"]):
        p = f"blk.{l}."
        h = orc.rmsnorm_into(x[0], v32(p + "attn_norm.weight"), eps)[None]
        q = heads(mm(p + "attn_q.weight", nq, H, h)[0], v32(p + "attn_q_norm.weight"))
        k = heads(mm(p + "attn_k.weight", nk, H, h)[0], v32(p + "attn_k_norm.weight"))
        v = mm(p + "attn_v.weight", nk, H, h)[0]
        kcs[l][pos], vcs[l][pos] = orc.kv_store(k), orc.kv_store(v)
        att = orc.attend_one(q, kcs[l], vcs[l], nk, nkv, hd, nh // nkv, 0, pos, scale)[None]
        x = x + mm(p + "attn_output.weight", H, nq, att)
        h = orc.rmsnorm_into(x[0], v32(p + "ffn_norm.weight"), eps)[None]
        g, u, d = (f.tensor(p + n) for n in ("ffn_gate.weight", "ffn_up.weight", "ffn_down.weight"))
        x = x + orc.ffn(g["ty"], g["data"], u["ty"], u["data"], d["ty"], d["data"], H, ffn, h, 1)
    head = f.tensor("output.weight") or f.tensor("token_embd.weight")
    return oracle_logits(orc, head["ty"], head["data"], info["vocab"], H, x, v32("output_norm.weight"), eps, 1)


# the Q4_K_M recipe: V, down and the embedding / head in Q6_K, the rest in Q4_K
K_M = {"attn_v.weight": Q6_K, "ffn_down.weight": Q6_K, "token_embd.weight": Q6_K, "output.weight": Q6_K}
# the Q5_K_M recipe: the same tensors in Q6_K, the rest in Q5_K


@pytest.mark.parametrize("arch,ty,tied,ty_of", [("qwen3", Q8_0, False, None), ("qwen3", Q4_K, True, None), ("qwen3", Q6_K, True, None),
                                                 ("llama", Q8_0, False, None), ("qwen3", Q4_K, True, K_M), ("llama", Q4_K, False, K_M), ("qwen3", Q5_K, True, K_M), ("qwen3", Q5_0, True, None), ("qwen3", Q3_K, True, None), ("qwen3", Q2_K, True, None)])
def test_tokens_from_a_model_file(orc, tmp_path, arch, ty, tied, ty_of):
    from allpaka_b200 import gpu as G

    pairwise = arch == "llama"
    meta, tensors = tiny_model(arch=arch, ty=ty, hidden=512, n_heads=4, n_kv=2, ffn=1024, vocab=1000, n_layers=2,
                               qk_norm=not pairwise, tied=tied, ty_of=ty_of)
    path = tmp_path / "model.gguf"
    gguf.write_file(str(path), meta, tensors)
    f = gguf.GgufFile(str(path))
    model = gguf.Model(f)
    info = model.info
    assert info["neox_reordered"] == (1 if pairwise else 0) and info["tied"] == (1 if tied else 0)
    g = G.Gpu(0)
    model.attach(g)
    cap = 16
    kv = G.KvCache(g, info["n_layers"], info["n_kv_heads"] * info["head_dim"], cap)
    kcs = [np.zeros((cap, info["n_kv_heads"] * info["head_dim"]), np.uint16) for _ in range(info["n_layers"])]
    vcs = [np.zeros_like(kcs[0]) for _ in range(info["n_layers"])]
    embd = f.tensor("token_embd.weight")["data"]
    rb = embd.size // info["vocab"]
    errs = []
    for pos, tok in enumerate((5, 999, 0, 128, 640)):
        req = model.request()
        rope = rope_table(orc, [pos], info["head_dim"], info["rot_dim"], info["rope_base"])
        req.rope = rope.ctypes.data
        req.token_id, req.use_token = tok, 1
        req.kv, req.pos = kv._h, pos
        got = g.decode_request(req)
        x = orc.dequant(f.tensor("token_embd.weight")["ty"], embd[tok * rb:(tok + 1) * rb], info["hidden"])
        want = oracle_step(orc, f, info, x, pos, kcs, vcs, pairwise)
        errs.append(rel_l2(got, want))
        assert int(np.argmax(got)) == int(np.argmax(want))
    print(f"{arch} file, ggml type {ty}{' (K_M mix)' if ty_of else ''}: logits rel-L2 per position " + " ".join(f"{e:.1e}" for e in errs))
    # The attention core's expf and the order of its sums differ from the CPU's by rounding, and a row
    # that lands on a rounding boundary of the Q8 activation codes moves one code (about 1e-3 of the
    # row, carried through the layers behind it): the typical position sits at rounding level, none may
    # leave the neighbourhood of the bar.
    assert np.median(errs) <= 2e-3 and max(errs) <= 2e-2
    kv.close()
    model.close()
    g.close()
    f.close()


def test_v_beside_qk_gives_the_same_logits(orc, tmp_path, monkeypatch):
    """In the K_M mix V has a type of its own and, for one token row, runs on SMs of its own beside the Q|K
    launch (a forked branch of the token graph).  ALLPAKA_B200_FORK_V=0 runs it after Q|K instead: the
    logits of a short decode must be the same bits either way."""
    from allpaka_b200 import gpu as G

    meta, tensors = tiny_model(arch="qwen3", ty=Q4_K, hidden=512, n_heads=4, n_kv=2, ffn=1024, vocab=1000, n_layers=3,
                               qk_norm=True, tied=True, ty_of=K_M)
    path = tmp_path / "model.gguf"
    gguf.write_file(str(path), meta, tensors)
    runs = []
    for fork in ("0", "4"):
        monkeypatch.setenv("ALLPAKA_B200_FORK_V", fork)
        f = gguf.GgufFile(str(path))
        model = gguf.Model(f)
        info = model.info
        g = G.Gpu(0)
        model.attach(g)
        kv = G.KvCache(g, info["n_layers"], info["n_kv_heads"] * info["head_dim"], 8)
        outs = []
        for pos, tok in enumerate((7, 400, 999, 3)):
            req = model.request()
            rope = rope_table(orc, [pos], info["head_dim"], info["rot_dim"], info["rope_base"])
            req.rope = rope.ctypes.data
            req.token_id, req.use_token = tok, 1
            req.kv, req.pos = kv._h, pos
            outs.append(np.array(g.decode_request(req)))
        runs.append(outs)
        kv.close()
        model.close()
        g.close()
        f.close()
    for a, b in zip(*runs):
        assert np.array_equal(a, b)

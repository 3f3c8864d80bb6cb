"""A model file end to end: GGUF written here -> reader -> model view -> attach -> tokens by id
through the decode path with the attention core and the f16 KV cache, against the oracle's
restatement of the same layer order on the file's own tensors."""
import numpy as np
import pytest

from allpaka_b200 import gguf
from tests.test_gguf_reader import tiny_model
from tests.util import Q4_K, Q6_K, Q8_0, oracle_logits, rel_l2, rope_table

pytestmark = pytest.mark.gpu


def rope_norm_rows(x, table, head_dim):
    """rope_norm_cached_from_array (ops/rope.rs:52-67) on every head of a row: pairs (2i, 2i+1)."""
    x = x.reshape(-1, head_dim).copy()
    for i, (sin, cos) in enumerate(table):
        a, b = x[:, 2 * i].copy(), x[:, 2 * i + 1].copy()
        x[:, 2 * i] = a * cos - b * sin
        x[:, 2 * i + 1] = a * sin + b * cos
    return x.reshape(-1)


def oracle_step(orc, f, info, ty, x, pos, kcs, vcs, pairwise):
    """One token through the file's layers (model/decode.rs:435-591 with model/attention.rs:78-330)."""
    H, hd, nh, nkv = info["hidden"], info["head_dim"], info["n_heads"], info["n_kv_heads"]
    nq, nk, ffn, eps = nh * hd, nkv * hd, info["ffn"], info["eps"]
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    inv = orc.rope_inv_freq(info["rot_dim"], info["rope_base"])
    table = orc.rope_sin_cos(pos, inv)

    def w(name):
        return f.tensor(name)["data"]

    def v32(name):
        t = f.tensor(name)
        return None if t is None else t["data"].view(np.float32)

    x = np.array(x, np.float32).reshape(1, H)
    for l in range(info["n_layers"]):
        p = f"blk.{l}."
        if pairwise:
            h = orc.rmsnorm_into(x[0], v32(p + "attn_norm.weight"), eps)[None]
            q = rope_norm_rows(orc.matmul(ty, w(p + "attn_q.weight"), nq, H, h, 1)[0], table, hd)[None]
            k = rope_norm_rows(orc.matmul(ty, w(p + "attn_k.weight"), nk, H, h, 1)[0], table, hd)[None]
            v = orc.matmul(ty, w(p + "attn_v.weight"), nk, H, h, 1)
        else:
            q, k, v = orc.attn_in(ty, w(p + "attn_q.weight"), w(p + "attn_k.weight"), w(p + "attn_v.weight"), H, nq, nk, hd, x, 1,
                                  v32(p + "attn_norm.weight"), eps, table[None], v32(p + "attn_q_norm.weight"),
                                  v32(p + "attn_k_norm.weight"))
        kcs[l][pos], vcs[l][pos] = orc.kv_store(k[0]), orc.kv_store(v[0])
        att = orc.attend_one(q[0], kcs[l], vcs[l], nk, nkv, hd, nh // nkv, 0, pos, scale)[None]
        x = x + orc.matmul(ty, w(p + "attn_output.weight"), H, nq, att, 1)
        h = orc.rmsnorm_into(x[0], v32(p + "ffn_norm.weight"), eps)[None]
        x = x + orc.ffn(ty, w(p + "ffn_gate.weight"), ty, w(p + "ffn_up.weight"), ty, w(p + "ffn_down.weight"), H, ffn, h, 1)
    head = w("output.weight") if f.tensor("output.weight") is not None else w("token_embd.weight")
    return oracle_logits(orc, ty, head, info["vocab"], H, x, v32("output_norm.weight"), eps, 1)


@pytest.mark.parametrize("arch,ty,tied", [("qwen3", Q8_0, False), ("qwen3", Q4_K, True), ("qwen3", Q6_K, True), ("llama", Q8_0, False)])
def test_tokens_from_a_model_file(orc, tmp_path, arch, ty, tied):
    from allpaka_b200 import gpu as G

    pairwise = arch == "llama"
    meta, tensors = tiny_model(arch=arch, ty=ty, hidden=512, n_heads=4, n_kv=2, ffn=1024, vocab=1000, n_layers=2,
                               qk_norm=not pairwise, tied=tied)
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
    worst = 0.0
    for pos, tok in enumerate((5, 999, 0, 128, 640)):
        req = model.request()
        rope = rope_table(orc, [pos], info["head_dim"], info["rot_dim"], info["rope_base"])
        req.rope = rope.ctypes.data
        req.token_id, req.use_token = tok, 1
        req.kv, req.pos = kv._h, pos
        got = g.decode_request(req)
        x = orc.dequant(ty, embd[tok * rb:(tok + 1) * rb], info["hidden"])
        want = oracle_step(orc, f, info, ty, x, pos, kcs, vcs, pairwise)
        worst = max(worst, rel_l2(got, want))
        assert int(np.argmax(got)) == int(np.argmax(want))
    print(f"{arch} file, ggml type {ty}: worst logits rel-L2 over 5 positions {worst:.1e}")
    assert worst <= 2e-3
    kv.close()
    model.close()
    g.close()
    f.close()

"""Shared helpers for the parity tests (test infrastructure)."""
import numpy as np

from allpaka_b200 import synth

Q8_0, Q4_K, Q5_K, Q6_K, Q5_0, Q3_K, Q2_K = 8, 12, 13, 14, 6, 11, 10


def rel_l2(got, want):
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    den = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / (den if den > 0 else 1.0))


def rope_table(orc, positions, head_dim, rot_dim, base=1e6):
    """Host-built (sin, cos) rows, one per token (ops/rope.rs:8-22)."""
    inv = orc.rope_inv_freq(rot_dim, base)
    return np.stack([orc.rope_sin_cos(int(p), inv) for p in positions]).astype(np.float32)


def make_layer(ty, hidden, n_q, n_kv, ffn, seed, qk_norm=False):
    L = {
        "wq": synth.matrix(ty, n_q, hidden, seed + 0),
        "wk": synth.matrix(ty, n_kv, hidden, seed + 1),
        "wv": synth.matrix(ty, n_kv, hidden, seed + 2),
        "wo": synth.matrix(ty, hidden, n_q, seed + 3),
        "gate": synth.matrix(ty, ffn, hidden, seed + 4),
        "up": synth.matrix(ty, ffn, hidden, seed + 5),
        "down": synth.matrix(ty, hidden, ffn, seed + 6),
        "attn_norm": synth.gamma(hidden, seed + 7),
        "ffn_norm": synth.gamma(hidden, seed + 8),
    }
    if qk_norm:
        L["q_norm"] = synth.gamma(128, seed + 9)
        L["k_norm"] = synth.gamma(128, seed + 10)
    return L


def oracle_decode(orc, ty, layers, hidden, n_q, n_kv, head_dim, ffn, eps, rope, x, m):
    """The reference's per-layer order for m rows with the identity attention
    core (model/decode.rs:435-591 at m = 1; model/prefill.rs batch path: QKV and
    gate/up through matmul_many, wo / down / head through matmul(., m))."""
    x = np.array(x, dtype=np.float32).reshape(m, hidden).copy()
    for L in layers:
        q, k, v = orc.attn_in(ty, L["wq"], L["wk"], L["wv"], hidden, n_q, n_kv, head_dim, x, m,
                              L["attn_norm"], eps, rope, L.get("q_norm"), L.get("k_norm"))
        x = x + orc.matmul(ty, L["wo"], hidden, n_q, q, m)
        h = np.stack([orc.rmsnorm_into(x[i], L["ffn_norm"], eps) for i in range(m)])
        x = x + orc.ffn(ty, L["gate"], ty, L["up"], ty, L["down"], hidden, ffn, h, m)
    return x


def oracle_logits(orc, ty, w, vocab, hidden, x, out_norm, eps, m):
    h = np.stack([orc.rmsnorm(np.asarray(x, np.float32).reshape(m, hidden)[i], out_norm, eps) for i in range(m)])
    return orc.matmul(ty, w, vocab, hidden, h, m)


class Region:
    """Weights packed back to back in one attached mapping, like tensors in a GGUF mmap."""

    def __init__(self, parts):
        sizes = [np.asarray(p).size for p in parts]
        offs = np.concatenate([[0], np.cumsum([(s + 63) // 64 * 64 for s in sizes])])
        self.buf = np.zeros(int(offs[-1]) + 64, dtype=np.uint8)
        self.views = []
        for p, o, s in zip(parts, offs, sizes):
            self.buf[o:o + s] = np.asarray(p).view(np.uint8).reshape(-1)
            self.views.append(self.buf[o:o + s])

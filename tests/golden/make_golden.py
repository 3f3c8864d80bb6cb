"""Regenerates tests/golden/*.npz from the CPU oracle.

The reference is Rust and cannot run where this is built, so these fixtures are
outputs of the oracle (itself pinned by the reference's known-answer tests) on
seeded inputs of the benchmark configurations, kept small: inputs are seeds,
outputs are stored in full only where they are small.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from allpaka_b200 import synth  # noqa: E402
from oracle import oracle as orc  # noqa: E402
from tests.util import make_layer, oracle_decode, oracle_logits, rope_table  # noqa: E402

Q8_0, Q4_K = 8, 12


def config0():
    """Q8_0 3072x1024, batch 1 (seed 1000)."""
    w = synth.q8_0_matrix(3072, 1024, 1000)
    x = synth.normal_f32(1024, 1001)
    d, s, q = orc.q8acts(x)
    dots = orc.block_dots(Q8_0, w, 3072, 1024, q)
    return dict(y=orc.matmul(Q8_0, w, 3072, 1024, x, 1)[0], q=q, d=d,
                dots_rowsum=dots[0].sum(axis=1).astype(np.int64), dots_head=dots[0, :8])


def q4k_small():
    """Q4_K 384x2048, batch 1 and 3."""
    w = synth.q4_k_matrix(384, 2048, 1100)
    x = synth.normal_f32((3, 2048), 1101)
    _, _, q = orc.q8acts(x[0])
    dots = orc.block_dots(Q4_K, w, 384, 2048, q)
    return dict(y1=orc.matmul(Q4_K, w, 384, 2048, x[0], 1)[0], y3_q8=orc.matmul(Q4_K, w, 384, 2048, x, 3, orc.ACT_Q8),
                y3_f32=orc.matmul(Q4_K, w, 384, 2048, x, 3, orc.ACT_F32), dots_rowsum=dots[0].sum(axis=1).astype(np.int64))


def attn_small():
    """RMSNorm -> Q|K|V -> per-head norm -> RoPE: hidden 1024, 4+2 heads of 128, m = 2, bf16 x."""
    hidden, nq, nk = 1024, 512, 256
    wq, wk, wv = (synth.q8_0_matrix(n, hidden, 1200 + i) for i, n in enumerate((nq, nk, nk)))
    _, x = synth.normal_bf16((2, hidden), 1203)
    rope = rope_table(orc, [31000, 7], 128, 128)
    q, k, v = orc.attn_in(Q8_0, wq, wk, wv, hidden, nq, nk, 128, x, 2, synth.gamma(hidden, 1204), 1e-6, rope,
                          synth.gamma(128, 1205), synth.gamma(128, 1206))
    return dict(q=q, k=k, v=v)


def ffn_small():
    """gate/up 2048x1024 + SwiGLU + down 1024x2048, m = 1 and 6."""
    hidden, ffn = 1024, 2048
    g, u, d = synth.q8_0_matrix(ffn, hidden, 1300), synth.q8_0_matrix(ffn, hidden, 1301), synth.q8_0_matrix(hidden, ffn, 1302)
    _, x = synth.normal_bf16((6, hidden), 1303)
    return dict(y1=orc.ffn(Q8_0, g, Q8_0, u, Q8_0, d, hidden, ffn, x[0], 1), y6=orc.ffn(Q8_0, g, Q8_0, u, Q8_0, d, hidden, ffn, x, 6))


def token_small():
    """Two decoder layers + head, hidden 512, m = 1."""
    hidden, nh, nkv, ffn, vocab = 512, 4, 2, 1024, 640
    layers = [make_layer(Q8_0, hidden, nh * 128, nkv * 128, ffn, 1400 + 100 * l, True) for l in range(2)]
    head = synth.q8_0_matrix(vocab, hidden, 1490)
    on = synth.gamma(hidden, 1491)
    x = synth.normal_f32((1, hidden), 1492)
    rope = rope_table(orc, [12345], 128, 128)
    xo = oracle_decode(orc, Q8_0, layers, hidden, nh * 128, nkv * 128, 128, ffn, 1e-6, rope, x, 1)
    return dict(hidden=xo, logits=oracle_logits(orc, Q8_0, head, vocab, hidden, xo, on, 1e-6, 1))


CASES = dict(config0=config0, q4k_small=q4k_small, attn_small=attn_small, ffn_small=ffn_small, token_small=token_small)

if __name__ == "__main__":
    orc.build()
    for name, fn in CASES.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **fn())
        print("wrote", name)

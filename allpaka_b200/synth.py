"""Seeded synthetic GGUF-layout tensors for tests and benchmarks.

The block layouts are the GGUF ones the engine reads from a model file
(crates/allpaka-dtype/src/lib.rs:93-108; crates/allpaka-gguf/src/dequant.rs:93-126,
206-231): Q8_0 = ``{f16 d; i8 q[32]}`` (34 B), Q4_K = ``{f16 d; f16 dmin;
u8 scales[12]; u8 qs[128]}`` (144 B), Q5_0 = ``{f16 d; u32 qh; u8 qs[16]}`` (22 B, dequant.rs:128-141), Q6_K = ``{u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d}``
(210 B, dequant.rs:265-296).  No model file is needed: the value
distributions below are the ones the benchmark configurations state.
"""
from __future__ import annotations

import numpy as np

TY_Q5_0 = 6
TY_Q2_K = 10
TY_Q3_K = 11
TY_Q8_0 = 8
TY_Q4_K = 12
TY_Q5_K = 13
TY_Q6_K = 14

BLOCK = {TY_Q8_0: (32, 34), TY_Q5_0: (32, 22), TY_Q2_K: (256, 84), TY_Q3_K: (256, 110), TY_Q4_K: (256, 144), TY_Q5_K: (256, 176), TY_Q6_K: (256, 210)}


def expected_bytes(ty: int, elements: int) -> int:
    be, bb = BLOCK[ty]
    if elements % be:
        raise ValueError(f"{elements} elements is not whole {be}-element blocks")
    return elements // be * bb


def q8_0_matrix(n_out: int, n_in: int, seed: int, scale_sigma: float = 0.02) -> np.ndarray:
    """int8 quants uniform in [-127,127], one f16 scale |N(0,sigma)|/127 per block."""
    rng = np.random.default_rng(seed)
    nb = n_in // 32
    out = np.empty((n_out, nb, 34), dtype=np.uint8)
    q = rng.integers(-127, 128, size=(n_out, nb, 32), dtype=np.int8)
    d = (np.abs(rng.normal(0.0, scale_sigma, size=(n_out, nb))) / 127.0).astype(np.float16)
    out[:, :, 0:2] = d.view(np.uint8).reshape(n_out, nb, 2)
    out[:, :, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def pack_scales_k4(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Pack 8 six-bit (scale, min) pairs into the 12-byte Q4_K/Q5_K field, the
    inverse of ``scale_min_k4`` (crates/allpaka-dtype/src/lib.rs:382-390)."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    p = np.zeros(sc.shape[:-1] + (12,), dtype=np.uint8)
    p[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    p[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    p[..., 8:12] = (sc[..., 4:8] & 0xF) | ((mn[..., 4:8] & 0xF) << 4)
    return p


def q4_k_matrix(n_out: int, n_in: int, seed: int, d_sigma: float = 0.002) -> np.ndarray:
    """4-bit quants uniform [0,15], 6-bit scales/mins uniform [0,63], f16 d and
    dmin drawn as |N(0,sigma)|."""
    rng = np.random.default_rng(seed)
    nsb = n_in // 256
    out = np.empty((n_out, nsb, 144), dtype=np.uint8)
    d = np.abs(rng.normal(0.0, d_sigma, size=(n_out, nsb))).astype(np.float16)
    dmin = np.abs(rng.normal(0.0, d_sigma, size=(n_out, nsb))).astype(np.float16)
    sc = rng.integers(0, 64, size=(n_out, nsb, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(n_out, nsb, 8), dtype=np.uint8)
    qs = rng.integers(0, 256, size=(n_out, nsb, 128), dtype=np.uint8)
    out[:, :, 0:2] = d.view(np.uint8).reshape(n_out, nsb, 2)
    out[:, :, 2:4] = dmin.view(np.uint8).reshape(n_out, nsb, 2)
    out[:, :, 4:16] = pack_scales_k4(sc, mn)
    out[:, :, 16:] = qs
    return out.reshape(-1)


def q5_k_matrix(n_out: int, n_in: int, seed: int, d_sigma: float = 0.001) -> np.ndarray:
    """Q5_K = ``{f16 d; f16 dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]}`` (176 B, dequant.rs:238-263):
    5-bit quants, 6-bit scales and mins uniform, d and dmin drawn as |N(0,sigma)|."""
    rng = np.random.default_rng(seed)
    nsb = n_in // 256
    out = np.empty((n_out, nsb, 176), dtype=np.uint8)
    d = np.abs(rng.normal(0.0, d_sigma, size=(n_out, nsb))).astype(np.float16)
    dmin = np.abs(rng.normal(0.0, d_sigma, size=(n_out, nsb))).astype(np.float16)
    sc = rng.integers(0, 64, size=(n_out, nsb, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(n_out, nsb, 8), dtype=np.uint8)
    out[:, :, 0:2] = d.view(np.uint8).reshape(n_out, nsb, 2)
    out[:, :, 2:4] = dmin.view(np.uint8).reshape(n_out, nsb, 2)
    out[:, :, 4:16] = pack_scales_k4(sc, mn)
    out[:, :, 16:] = rng.integers(0, 256, size=(n_out, nsb, 160), dtype=np.uint8)
    return out.reshape(-1)


def q6_k_matrix(n_out: int, n_in: int, seed: int, d_sigma: float = 2.5e-5) -> np.ndarray:
    """6-bit quants uniform (every ql/qh byte uniform), signed 8-bit sub-block scales uniform in
    [-128,127], f16 d drawn as |N(0,sigma)|: weights of a few hundredths, like a model's (d of a
    real file, max|w| / (127 * 32), lies in the f16 subnormal range too)."""
    rng = np.random.default_rng(seed)
    nsb = n_in // 256
    out = np.empty((n_out, nsb, 210), dtype=np.uint8)
    out[:, :, 0:192] = rng.integers(0, 256, size=(n_out, nsb, 192), dtype=np.uint8)
    out[:, :, 192:208] = rng.integers(-128, 128, size=(n_out, nsb, 16), dtype=np.int8).view(np.uint8)
    d = np.abs(rng.normal(0.0, d_sigma, size=(n_out, nsb))).astype(np.float16)
    out[:, :, 208:210] = d.view(np.uint8).reshape(n_out, nsb, 2)
    return out.reshape(-1)


def q5_0_matrix(n_out: int, n_in: int, seed: int, scale_sigma: float = 0.02) -> np.ndarray:
    """5-bit quants uniform in [0,31] (value q - 16), one f16 scale |N(0,sigma)|/15 per block."""
    rng = np.random.default_rng(seed)
    nb = n_in // 32
    out = np.empty((n_out, nb, 22), dtype=np.uint8)
    d = (np.abs(rng.normal(0.0, scale_sigma, size=(n_out, nb))) / 15.0).astype(np.float16)
    out[:, :, 0:2] = d.view(np.uint8).reshape(n_out, nb, 2)
    out[:, :, 2:] = rng.integers(0, 256, size=(n_out, nb, 20), dtype=np.uint8)
    return out.reshape(-1)


def q3_k_matrix(n_out: int, n_in: int, seed: int, d_sigma: float = 1e-4) -> np.ndarray:
    """Q3_K = ``{u8 hmask[32]; u8 qs[64]; u8 scales[12]; f16 d}`` (110 B, dequant.rs:176-204): uniform
    masks, 2-bit quants and packed 6-bit scales, d ~ |N(0, d_sigma)| (value = d * (scale - 32) * q with
    q in [-4, 3])."""
    rng = np.random.default_rng(seed)
    nsb = n_in // 256
    out = np.empty((n_out, nsb, 110), dtype=np.uint8)
    out[:, :, 0:108] = rng.integers(0, 256, size=(n_out, nsb, 108), dtype=np.uint8)
    d = np.abs(rng.normal(0.0, d_sigma, size=(n_out, nsb))).astype(np.float16)
    out[:, :, 108:110] = d.view(np.uint8).reshape(n_out, nsb, 2)
    return out.reshape(-1)


def q2_k_matrix(n_out: int, n_in: int, seed: int, d_sigma: float = 4e-4) -> np.ndarray:
    """Q2_K = ``{u8 scales[16]; u8 qs[64]; f16 d; f16 dmin}`` (84 B, dequant.rs:143-174): uniform packed
    4-bit scales / mins and 2-bit quants, d and dmin ~ |N(0, d_sigma)|."""
    rng = np.random.default_rng(seed)
    nsb = n_in // 256
    out = np.empty((n_out, nsb, 84), dtype=np.uint8)
    out[:, :, 0:80] = rng.integers(0, 256, size=(n_out, nsb, 80), dtype=np.uint8)
    dd = np.abs(rng.normal(0.0, d_sigma, size=(n_out, nsb, 2))).astype(np.float16)
    out[:, :, 80:84] = dd.view(np.uint8).reshape(n_out, nsb, 4)
    return out.reshape(-1)


def matrix(ty: int, n_out: int, n_in: int, seed: int) -> np.ndarray:
    if ty == TY_Q2_K:
        return q2_k_matrix(n_out, n_in, seed)
    if ty == TY_Q3_K:
        return q3_k_matrix(n_out, n_in, seed)
    if ty == TY_Q8_0:
        return q8_0_matrix(n_out, n_in, seed)
    if ty == TY_Q5_0:
        return q5_0_matrix(n_out, n_in, seed)
    if ty == TY_Q4_K:
        return q4_k_matrix(n_out, n_in, seed)
    if ty == TY_Q5_K:
        return q5_k_matrix(n_out, n_in, seed)
    if ty == TY_Q6_K:
        return q6_k_matrix(n_out, n_in, seed)
    raise ValueError(f"no generator for ggml type {ty}")


def normal_f32(shape, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (b & 0x7FFFFFFF) > 0x7F800000
    r = ((b + (0x7FFF + ((b >> 16) & 1))) >> 16).astype(np.uint16)
    r[nan] = ((b[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    return (h.astype(np.uint32) << 16).view(np.float32)


def normal_bf16(shape, seed: int):
    """N(0,1) rounded to bf16: returns (bits uint16, the same values widened to f32)."""
    bits = to_bf16_bits(normal_f32(shape, seed))
    return bits, bf16_bits_to_f32(bits)


def gamma(n: int, seed: int) -> np.ndarray:
    return (1.0 + 0.1 * np.random.default_rng(seed).standard_normal(n)).astype(np.float32)


def lcg_bytes(n: int, state: int) -> np.ndarray:
    """The 64-bit LCG the engine's own tests fill weight regions with, top byte
    of each state (crates/allpaka-backend/src/quantmat/kernel_tests.rs:13-23)."""
    out = np.empty(n, dtype=np.uint8)
    mask = (1 << 64) - 1
    for i in range(n):
        state = (state * 6364136223846793005 + 1442695040888963407) & mask
        out[i] = state >> 56
    return out


def tame_scales(buf: np.ndarray, ty: int, value: int = 0x211F) -> np.ndarray:
    """Overwrite every f16 scale field with ~0.01 so random bytes decode to
    finite numbers (crates/allpaka-backend/tests/gpu_cuda_parity.rs:58-70)."""
    be, bb = BLOCK[ty]
    v = buf.reshape(-1, bb)
    lo, hi = value & 0xFF, value >> 8
    offs = {TY_Q8_0: (0,), TY_Q5_0: (0,), TY_Q2_K: (80, 82), TY_Q3_K: (108,), TY_Q4_K: (0, 2), TY_Q5_K: (0, 2), TY_Q6_K: (208,)}[ty]
    for o in offs:
        v[:, o] = lo
        v[:, o + 1] = hi
    return buf

"""ctypes binding of the CPU oracle (``libapk_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()``
and ``bench.py``'s CPU-baseline legs, never by the product package.  The
library restates the reference's CPU arithmetic for the decode dequant-matvec
path (citations live in ``apk_oracle.h`` / ``apk_oracle.c``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libapk_oracle.so")

TY_Q8_0 = 8
TY_Q5_0 = 6
TY_Q2_K = 10
TY_Q3_K = 11
TY_Q4_K = 12
TY_Q5_K = 13
TY_Q6_K = 14
ACT_Q8, ACT_F32, ACT_AUTO = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc only)."""
    src = [os.path.join(_HERE, f) for f in ("apk_oracle.c", "apk_oracle.h", "Makefile")]
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src
    )
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "libapk_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)
_i32p = C.POINTER(C.c_int32)


class _Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("wq", "wk", "wv", "wo", "gate", "up", "down", "attn_norm", "ffn_norm",
                 "q_norm", "k_norm")]


def _declare(l):
    l.orc_f16_to_f32.restype = C.c_float
    l.orc_f16_to_f32.argtypes = [C.c_uint16]
    l.orc_f32_to_f16.restype = C.c_uint16
    l.orc_f32_to_f16.argtypes = [C.c_float]
    l.orc_bf16_to_f32.restype = C.c_float
    l.orc_bf16_to_f32.argtypes = [C.c_uint16]
    l.orc_f32_to_bf16.restype = C.c_uint16
    l.orc_f32_to_bf16.argtypes = [C.c_float]
    l.orc_scale_min_k4.restype = None
    l.orc_scale_min_k4.argtypes = [C.c_int, C.c_void_p, _f32p, _f32p]
    l.orc_expected_bytes.restype = C.c_size_t
    l.orc_expected_bytes.argtypes = [C.c_uint32, C.c_size_t]
    l.orc_dequant.restype = C.c_int
    l.orc_dequant.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]
    l.orc_q8acts_from_f32.restype = None
    l.orc_q8acts_from_f32.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]
    l.orc_dot_i8.restype = C.c_int32
    l.orc_dot_i8.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    for name in ("orc_dot_q8_0_i8",):
        getattr(l, name).restype = C.c_float
        getattr(l, name).argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    l.orc_dot_q4_k_i8.restype = C.c_float
    l.orc_dot_q4_k_i8.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]
    l.orc_dot_q5_k_i8.restype = C.c_float
    l.orc_dot_q5_k_i8.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]
    l.orc_dot_q6_k_i8.restype = C.c_float
    l.orc_dot_q6_k_i8.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    l.orc_dot_q5_0_i8.restype = C.c_float
    l.orc_dot_q5_0_i8.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    l.orc_dot_q3_k_i8.restype = C.c_float
    l.orc_dot_q3_k_i8.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    l.orc_dot_q2_k_i8.restype = C.c_float
    l.orc_dot_q2_k_i8.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    for name in ("orc_dot_q8_0", "orc_dot_q5_0", "orc_dot_q3_k", "orc_dot_q2_k", "orc_dot_q4_k", "orc_dot_q5_k", "orc_dot_q6_k"):
        getattr(l, name).restype = C.c_float
        getattr(l, name).argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
    l.orc_block_dots.restype = C.c_int
    l.orc_block_dots.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                                 C.c_size_t, C.c_void_p]
    l.orc_matmul.restype = C.c_int
    l.orc_matmul.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                             C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_int]
    l.orc_sum_sq_f64.restype = C.c_double
    l.orc_sum_sq_f64.argtypes = [C.c_void_p, C.c_size_t]
    l.orc_rmsnorm.restype = None
    l.orc_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_float]
    l.orc_rmsnorm_into.restype = None
    l.orc_rmsnorm_into.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_float]
    l.orc_rope_inv_freq.restype = None
    l.orc_rope_inv_freq.argtypes = [C.c_size_t, C.c_float, C.c_void_p]
    l.orc_rope_sin_cos.restype = None
    l.orc_rope_sin_cos.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_void_p]
    l.orc_rope_neox_table.restype = None
    l.orc_rope_neox_table.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]
    l.orc_rope_neox.restype = None
    l.orc_rope_neox.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32, C.c_float]
    l.orc_silu.restype = C.c_float
    l.orc_silu.argtypes = [C.c_float]
    l.orc_swiglu.restype = None
    l.orc_swiglu.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    l.orc_attn_in.restype = C.c_int
    l.orc_attn_in.argtypes = [C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                              C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t,
                              C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p,
                              C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    l.orc_ffn.restype = C.c_int
    l.orc_ffn.argtypes = [C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p,
                          C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p,
                          C.c_int]
    l.orc_decode_layers.restype = C.c_int
    l.orc_decode_layers.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                    C.c_size_t, C.c_size_t, C.c_size_t, C.c_float, C.c_void_p,
                                    C.c_size_t, C.c_void_p, C.c_int]
    l.orc_kv_store.restype = None
    l.orc_kv_store.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
    l.orc_attend_one.restype = None
    l.orc_attend_one.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                 C.c_size_t, C.c_size_t, C.c_float, C.c_void_p]
    l.orc_attend_head.restype = None
    l.orc_attend_head.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                  C.c_float, C.c_void_p]
    l.orc_lm_head.restype = C.c_int
    l.orc_lm_head.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                              C.c_void_p, C.c_float, C.c_void_p, C.c_int]
    l.orc_cpu_threads.restype = C.c_int
    l.orc_cpu_threads.argtypes = []


def _p(a):
    return None if a is None else a.ctypes.data


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


# ------------------------------------------------------------------ scalars

def f16_to_f32(h: int) -> float:
    return lib().orc_f16_to_f32(int(h) & 0xFFFF)


def f32_to_f16(x: float) -> int:
    return lib().orc_f32_to_f16(float(x))


def bf16_to_f32(h: int) -> float:
    return lib().orc_bf16_to_f32(int(h) & 0xFFFF)


def f32_to_bf16(x: float) -> int:
    return lib().orc_f32_to_bf16(float(x))


def scale_min_k4(j: int, packed) -> tuple[float, float]:
    packed = _u8(packed)
    sc, mn = C.c_float(), C.c_float()
    lib().orc_scale_min_k4(j, _p(packed), C.byref(sc), C.byref(mn))
    return sc.value, mn.value


def expected_bytes(ty: int, elements: int) -> int:
    return lib().orc_expected_bytes(ty, elements)


def cpu_threads() -> int:
    return lib().orc_cpu_threads()


# ------------------------------------------------------------------- arrays

def dequant(ty: int, data, n: int) -> np.ndarray:
    data = _u8(data)
    out = np.empty(n, dtype=np.float32)
    if lib().orc_dequant(ty, _p(data), data.size, _p(out), n) != 0:
        raise ValueError(f"dequant: bad type {ty} or byte count {data.size} for {n} elements")
    return out


def q8acts(x):
    """Q8Acts::from_f32 over the flattened x: returns (d, sum, q)."""
    x = _f32(x).reshape(-1)
    if x.size % 32:
        raise ValueError("activation length must be whole 32-element blocks")
    d = np.empty(x.size // 32, dtype=np.float32)
    s = np.empty(x.size // 32, dtype=np.float32)
    q = np.empty(x.size, dtype=np.int8)
    lib().orc_q8acts_from_f32(_p(x), x.size, _p(d), _p(s), _p(q))
    return d, s, q


def dot_i8(a, b) -> int:
    a = np.ascontiguousarray(a, dtype=np.int8)
    b = np.ascontiguousarray(b, dtype=np.int8)
    assert a.size == b.size
    return lib().orc_dot_i8(_p(a), _p(b), a.size)


def dot_row(ty: int, row, x, q8: bool) -> float:
    """One weight row against one activation row (f32 or Q8-activation path)."""
    row = _u8(row)
    x = _f32(x).reshape(-1)
    n_in = x.size
    l = lib()
    if q8:
        d, s, q = q8acts(x)
        if ty == TY_Q8_0:
            return l.orc_dot_q8_0_i8(_p(row), n_in, _p(d), _p(q))
        if ty == TY_Q6_K:
            return l.orc_dot_q6_k_i8(_p(row), n_in, _p(d), _p(q))
        if ty == TY_Q5_0:
            return l.orc_dot_q5_0_i8(_p(row), n_in, _p(d), _p(q))
        if ty == TY_Q3_K:
            return l.orc_dot_q3_k_i8(_p(row), n_in, _p(d), _p(q))
        if ty == TY_Q2_K:
            return l.orc_dot_q2_k_i8(_p(row), n_in, _p(d), _p(q))
        if ty == TY_Q5_K:
            return l.orc_dot_q5_k_i8(_p(row), n_in, _p(d), _p(s), _p(q))
        return l.orc_dot_q4_k_i8(_p(row), n_in, _p(d), _p(s), _p(q))
    fn = {TY_Q8_0: l.orc_dot_q8_0, TY_Q5_0: l.orc_dot_q5_0, TY_Q3_K: l.orc_dot_q3_k, TY_Q2_K: l.orc_dot_q2_k, TY_Q4_K: l.orc_dot_q4_k, TY_Q5_K: l.orc_dot_q5_k, TY_Q6_K: l.orc_dot_q6_k}[ty]
    return fn(_p(row), n_in, _p(x))


def block_dots(ty: int, w, n_out: int, n_in: int, q, m: int = 1) -> np.ndarray:
    w = _u8(w)
    q = np.ascontiguousarray(q, dtype=np.int8).reshape(-1)
    out = np.empty((m, n_out, n_in // 32), dtype=np.int32)
    if lib().orc_block_dots(ty, _p(w), n_out, n_in, _p(q), m, _p(out)) != 0:
        raise ValueError("block_dots: bad geometry")
    return out


def matmul(ty: int, w, n_out: int, n_in: int, x, m: int = 1, act_mode: int = ACT_AUTO,
           threads: int = 0) -> np.ndarray:
    """QuantMat::matmul (ACT_AUTO) or the matmul_many row rule (ACT_Q8)."""
    w = _u8(w)
    x = _f32(x).reshape(-1)
    if x.size != m * n_in:
        raise ValueError(f"x has {x.size} values, expected {m} x {n_in}")
    y = np.empty((m, n_out), dtype=np.float32)
    if lib().orc_matmul(ty, _p(w), w.size, n_out, n_in, _p(x), m, act_mode, _p(y), threads) != 0:
        raise ValueError(f"{n_out}x{n_in} of type {ty}: geometry / byte count mismatch ({w.size})")
    return y


def sum_sq_f64(x) -> float:
    x = _f32(x).reshape(-1)
    return lib().orc_sum_sq_f64(_p(x), x.size)


def rmsnorm(x, w, eps: float) -> np.ndarray:
    x = _f32(x).reshape(-1).copy()
    w = _f32(w).reshape(-1)
    assert x.size == w.size
    lib().orc_rmsnorm(_p(x), _p(w), x.size, eps)
    return x


def rmsnorm_into(x, w, eps: float) -> np.ndarray:
    x = _f32(x).reshape(-1)
    w = _f32(w).reshape(-1)
    assert x.size == w.size
    out = np.empty_like(x)
    lib().orc_rmsnorm_into(_p(out), _p(x), _p(w), x.size, eps)
    return out


def rope_inv_freq(head_dim: int, base: float) -> np.ndarray:
    out = np.empty(head_dim // 2, dtype=np.float32)
    lib().orc_rope_inv_freq(head_dim, base, _p(out))
    return out


def rope_sin_cos(pos: int, inv_freq) -> np.ndarray:
    inv_freq = _f32(inv_freq)
    out = np.empty((inv_freq.size, 2), dtype=np.float32)
    lib().orc_rope_sin_cos(pos, _p(inv_freq), inv_freq.size, _p(out))
    return out


def rope_neox_table(x, table) -> np.ndarray:
    x = _f32(x).reshape(-1).copy()
    table = _f32(table).reshape(-1, 2)
    lib().orc_rope_neox_table(_p(x), x.size, _p(table), table.shape[0])
    return x


def rope_neox(x, pos: int, base: float) -> np.ndarray:
    x = _f32(x).reshape(-1).copy()
    lib().orc_rope_neox(_p(x), x.size, pos, base)
    return x


def silu(x: float) -> float:
    return lib().orc_silu(float(x))


def swiglu(gate, up) -> np.ndarray:
    g = _f32(gate).reshape(-1).copy()
    u = _f32(up).reshape(-1)
    assert g.size == u.size
    lib().orc_swiglu(_p(g), _p(u), g.size)
    return g


def attn_in(ty, wq, wk, wv, hidden, n_q, n_kv, head_dim, x, m, gamma, eps, rope,
            q_norm=None, k_norm=None, threads=0):
    wq, wk, wv = _u8(wq), _u8(wk), _u8(wv)
    x = _f32(x).reshape(-1)
    gamma = None if gamma is None else _f32(gamma)
    q_norm = None if q_norm is None else _f32(q_norm)
    k_norm = None if k_norm is None else _f32(k_norm)
    rope = _f32(rope).reshape(m, -1, 2)
    half = rope.shape[1]
    q = np.empty((m, n_q), dtype=np.float32)
    k = np.empty((m, n_kv), dtype=np.float32)
    v = np.empty((m, n_kv), dtype=np.float32)
    rc = lib().orc_attn_in(ty, _p(wq), _p(wk), _p(wv), hidden, n_q, n_kv, head_dim, _p(x), m,
                           _p(gamma), eps, _p(q_norm), _p(k_norm), _p(rope), half,
                           _p(q), _p(k), _p(v), threads)
    if rc:
        raise ValueError("attn_in: geometry mismatch")
    return q, k, v


def ffn(gate_ty, gate, up_ty, up, down_ty, down, hidden, ffn_dim, x, m, threads=0,
        return_act=False):
    gate, up, down = _u8(gate), _u8(up), _u8(down)
    x = _f32(x).reshape(-1)
    y = np.empty((m, hidden), dtype=np.float32)
    act = np.empty((m, ffn_dim), dtype=np.float32) if return_act else None
    rc = lib().orc_ffn(gate_ty, _p(gate), up_ty, _p(up), down_ty, _p(down), hidden, ffn_dim,
                       _p(x), m, _p(y), _p(act), threads)
    if rc:
        raise ValueError("ffn: geometry mismatch")
    return (y, act) if return_act else y


def decode_layers(ty, layers, hidden, n_q, n_kv, head_dim, ffn_dim, eps, rope, x, threads=0):
    """layers: list of dicts with uint8 wq/wk/wv/wo/gate/up/down and f32
    attn_norm/ffn_norm (+ optional q_norm/k_norm).  Returns the updated x."""
    arr = (_Layer * len(layers))()
    keep = []
    for i, L in enumerate(layers):
        for name, _ in _Layer._fields_:
            v = L.get(name)
            if v is None:
                setattr(arr[i], name, None)
                continue
            v = _u8(v) if name in ("wq", "wk", "wv", "wo", "gate", "up", "down") else _f32(v)
            keep.append(v)
            setattr(arr[i], name, v.ctypes.data)
    rope = _f32(rope).reshape(-1, 2)
    x = _f32(x).reshape(-1).copy()
    rc = lib().orc_decode_layers(ty, C.addressof(arr), len(layers), hidden, n_q, n_kv, head_dim,
                                 ffn_dim, eps, _p(rope), rope.shape[0], _p(x), threads)
    if rc:
        raise ValueError("decode_layers: geometry mismatch")
    return x


def lm_head(ty, w, vocab, hidden, x, output_norm, eps, threads=0):
    w = _u8(w)
    x = _f32(x).reshape(-1)
    g = _f32(output_norm)
    out = np.empty(vocab, dtype=np.float32)
    if lib().orc_lm_head(ty, _p(w), vocab, hidden, _p(x), _p(g), eps, _p(out), threads):
        raise ValueError("lm_head: geometry mismatch")
    return out


def kv_store(row) -> np.ndarray:
    """f32 -> f16 bits, round to nearest even, as KvCache::store_at keeps K and V (model/kv.rs:695-696)."""
    row = _f32(row).reshape(-1)
    out = np.empty(row.size, dtype=np.uint16)
    lib().orc_kv_store(_p(row), row.size, _p(out))
    return out


def attend_one(q_row, kcache, vcache, kv_dim, n_kv_heads, head_dim, group, first, pos, scale) -> np.ndarray:
    """All heads of one row over cache positions first..=pos (model/attention.rs:403-428, 337-399).
    kcache / vcache: one layer's [capacity, kv_dim] uint16 (f16 bits)."""
    q_row = _f32(q_row).reshape(-1)
    kc = np.ascontiguousarray(kcache, dtype=np.uint16)
    vc = np.ascontiguousarray(vcache, dtype=np.uint16)
    out = np.zeros(n_kv_heads * group * head_dim, dtype=np.float32)
    lib().orc_attend_one(_p(q_row), _p(kc), _p(vc), kv_dim, n_kv_heads, head_dim, group, first, pos, scale, _p(out))
    return out


def attend_head(qh, kcache, vcache, kv_dim, kv_head, head_dim, pos, scale) -> np.ndarray:
    """The naive one-head formulation (model/attention.rs:430-465)."""
    qh = _f32(qh).reshape(-1)
    kc = np.ascontiguousarray(kcache, dtype=np.uint16)
    vc = np.ascontiguousarray(vcache, dtype=np.uint16)
    out = np.zeros(head_dim, dtype=np.float32)
    lib().orc_attend_head(_p(qh), _p(kc), _p(vc), kv_dim, kv_head, head_dim, pos, scale, _p(out))
    return out

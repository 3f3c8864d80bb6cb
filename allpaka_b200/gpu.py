"""Host-side mirror of allpaka-backend's accelerator module (``crate::gpu``).

Same free-function surface, names and argument meaning as the module every
reference backend implements (crates/allpaka-backend/src/gpu/stub.rs:37-217;
request structs gpu/types.rs:9-31, 54-80, 111-252): ``attach``, ``detach``,
``is_attached``, ``matvec``, ``matvec_batch``, ``ffn_batch``, ``attn_block``'s
input half, ``decode_token_checked`` / ``decode_token``, ``stats``,
``decode_path_stats``.  A declined request returns ``None`` (Rust ``Option``);
``decode_token_checked`` raises :class:`DecodeDecline`; hard errors raise
:class:`GpuError`.  Everything runs through the C ABI of ``libapk_b200.so``;
there is no CPU path here, and a missing library is an error, not a fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libapk_b200.so")

# GGML type ids (crates/allpaka-dtype/src/lib.rs:61-75)
Q8_0 = 8
Q4_K = 12
Q5_0 = 6
Q2_K = 10
Q3_K = 11
Q5_K = 13
Q6_K = 14

ACT_Q8, ACT_F32, ACT_AUTO = 0, 1, 2
ATTN_IDENTITY = 1
ATTN_CAUSAL = 2
MAX_M = 8

_DECLINE_NAMES = {
    1: "NoDevice", 2: "UnsupportedTensorType", 3: "UnsupportedShape", 4: "ForeignMemory",
    5: "MissingCapability", 6: "InvalidState", 7: "Backend",
}


class GpuError(RuntimeError):
    """A hard failure (CUDA/NCCL error, expired device wait, invalid argument)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"apk error {code}: {message}")
        self.code = code


class DecodeDecline(Exception):
    """``DecodeDecline { stage, reason }`` (gpu/types.rs:240-252)."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code
        self.reason = _DECLINE_NAMES.get(code, str(code))


class _MatvecReq(C.Structure):
    _fields_ = [("ty", C.c_uint32), ("w", C.c_void_p), ("n_in", C.c_uint32), ("n_out", C.c_uint32),
                ("x", C.c_void_p), ("m", C.c_uint32)]


class _FfnReq(C.Structure):
    _fields_ = [("gate_ty", C.c_uint32), ("gate_w", C.c_void_p), ("up_ty", C.c_uint32),
                ("up_w", C.c_void_p), ("down_ty", C.c_uint32), ("down_w", C.c_void_p),
                ("hidden", C.c_uint32), ("ffn", C.c_uint32), ("x", C.c_void_p), ("m", C.c_uint32)]


class _AttnInReq(C.Structure):
    _fields_ = [("ty", C.c_uint32), ("wq", C.c_void_p), ("wk", C.c_void_p), ("wv", C.c_void_p),
                ("hidden", C.c_uint32), ("head_dim", C.c_uint32), ("n_heads", C.c_uint32),
                ("n_kv_heads", C.c_uint32), ("x", C.c_void_p), ("m", C.c_uint32),
                ("gamma", C.c_void_p), ("eps", C.c_float), ("q_norm", C.c_void_p),
                ("k_norm", C.c_void_p), ("rope", C.c_void_p), ("rot_dim", C.c_uint32)]


class _Mat(C.Structure):
    _fields_ = [("ty", C.c_uint32), ("w", C.c_void_p), ("n_out", C.c_uint32)]


class _TokenLayer(C.Structure):
    _fields_ = [("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p),
                ("wq", _Mat), ("wk", _Mat), ("wv", _Mat), ("wo", _Mat),
                ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("gate", _Mat), ("up", _Mat), ("down", _Mat)]


class _TokenReq(C.Structure):
    _fields_ = [("layers", C.c_void_p), ("n_layers", C.c_uint32), ("output_norm", C.c_void_p),
                ("output", _Mat), ("x", C.c_void_p), ("m", C.c_uint32), ("rope", C.c_void_p),
                ("rot_dim", C.c_uint32), ("eps", C.c_float), ("hidden", C.c_uint32),
                ("head_dim", C.c_uint32), ("n_heads", C.c_uint32), ("n_kv_heads", C.c_uint32),
                ("attn_core", C.c_uint32), ("argmax", C.c_int),
                ("embd", _Mat), ("token_id", C.c_uint32), ("use_token", C.c_int),
                ("kv", C.c_void_p), ("pos", C.c_uint32), ("scale", C.c_float)]


class _TokenOut(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("argmax", C.c_void_p), ("hidden", C.c_void_p)]


class _BenchReq(C.Structure):
    _fields_ = [("op", C.c_uint32), ("n_copies", C.c_uint32), ("mv", C.c_void_p), ("attn", C.c_void_p),
                ("ffn", C.c_void_p), ("act_mode", C.c_uint32)]


class _Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in
                ("calls", "launches", "encode_ns", "wait_ns", "weight_bytes",
                 "decode_attempts", "decode_successes", "decode_declines")]


EXPORTS = (
    "apk_init", "apk_shutdown", "apk_attach", "apk_detach", "apk_is_attached",
    "apk_register_matrix", "apk_matvec", "apk_matvec_batch", "apk_ffn", "apk_attn_in",
    "apk_decode_token", "apk_decode_replay", "apk_debug_block_dots", "apk_debug_q8_acts",
    "apk_stats", "apk_last_error", "apk_dist_unique_id", "apk_dist_init",
    "apk_debug_synth_matrix", "apk_debug_synth_release", "apk_decode_profile",
    "apk_debug_matvec_timeline", "apk_shard_plan", "apk_matvec_noalloc",
    "apk_dist_p2p_export", "apk_dist_p2p_open", "apk_debug_token_timeline",
    "apk_debug_token_records", "apk_debug_set_wait_limit", "apk_debug_xch_timeout",
    "apk_bench_ring", "apk_dist_set_exchange", "apk_decode_greedy",
    "apk_kv_create", "apk_kv_destroy", "apk_kv_read", "apk_kv_write", "apk_attend", "apk_bench_attend",
    "apk_gguf_open", "apk_gguf_close", "apk_gguf_n_tensors", "apk_gguf_tensor_at", "apk_gguf_find",
    "apk_gguf_architecture", "apk_gguf_meta_u32", "apk_gguf_meta_f32", "apk_gguf_meta_str", "apk_gguf_mapping",
    "apk_model_open", "apk_model_get_info", "apk_model_token_req", "apk_model_attach", "apk_model_close",
)

_lib = None


def load_library() -> C.CDLL:
    """dlopen libapk_b200.so; a missing library is a hard error."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise GpuError(-1, f"{LIB_PATH} is missing: build it with `python -m allpaka_b200.build` "
                           "(there is no CPU fallback)")
    l = C.CDLL(LIB_PATH)
    l.apk_init.argtypes = [C.POINTER(C.c_void_p), C.c_int]
    l.apk_shutdown.argtypes = [C.c_void_p]
    l.apk_shutdown.restype = None
    l.apk_attach.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    l.apk_detach.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    l.apk_is_attached.argtypes = [C.c_void_p]
    l.apk_register_matrix.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32]
    l.apk_matvec.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                             C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p]
    l.apk_matvec_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p]
    l.apk_ffn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    l.apk_attn_in.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    l.apk_decode_token.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    l.apk_decode_replay.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(C.c_float)]
    l.apk_decode_greedy.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
    l.apk_kv_create.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_void_p)]
    l.apk_kv_destroy.argtypes = [C.c_void_p, C.c_void_p]
    l.apk_kv_destroy.restype = None
    l.apk_kv_read.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
    l.apk_kv_write.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
    l.apk_bench_attend.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_uint32,
                                   C.POINTER(C.c_float)]
    l.apk_attend.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float,
                             C.c_void_p]
    l.apk_debug_block_dots.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                       C.c_void_p, C.c_uint32, C.c_void_p]
    l.apk_debug_q8_acts.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_float,
                                    C.c_void_p, C.c_void_p, C.c_void_p]
    l.apk_debug_synth_matrix.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                         C.c_uint64, C.c_int]
    l.apk_debug_synth_release.argtypes = [C.c_void_p]
    l.apk_debug_matvec_timeline.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p,
                                            C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p]
    l.apk_debug_token_timeline.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
    l.apk_debug_token_records.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t]
    l.apk_debug_set_wait_limit.argtypes = [C.c_void_p, C.c_uint64]
    l.apk_debug_xch_timeout.argtypes = [C.c_void_p]
    l.apk_bench_ring.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(C.c_float)]
    l.apk_dist_set_exchange.argtypes = [C.c_void_p, C.c_int]
    l.apk_matvec_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p,
                                     C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_int]
    l.apk_decode_profile.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
    l.apk_stats.argtypes = [C.c_void_p, C.c_void_p]
    l.apk_stats.restype = None
    l.apk_last_error.argtypes = [C.c_void_p]
    l.apk_last_error.restype = C.c_char_p
    l.apk_shard_plan.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, C.c_int,
                                 C.c_void_p]
    l.apk_dist_p2p_export.argtypes = [C.c_void_p, C.c_void_p]
    l.apk_dist_p2p_open.argtypes = [C.c_void_p, C.c_void_p]
    l.apk_dist_unique_id.argtypes = [C.c_void_p]
    l.apk_dist_init.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    _lib = l
    return l


def _u8(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a) -> Optional[int]:
    return None if a is None else a.ctypes.data


@dataclass
class MatvecReq:
    """gpu/types.rs:9-16"""
    ty: int
    w: np.ndarray
    n_in: int
    n_out: int
    x: np.ndarray
    m: int


@dataclass
class FfnReq:
    """gpu/types.rs:20-31"""
    gate_ty: int
    gate_w: np.ndarray
    up_ty: int
    up_w: np.ndarray
    down_ty: int
    down_w: np.ndarray
    hidden: int
    ffn: int
    x: np.ndarray
    m: int


@dataclass
class TokenLayer:
    """gpu/types.rs:111-150, dense attention layers; matrices are (ty, bytes, n_out)."""
    attn_norm: np.ndarray
    ffn_norm: np.ndarray
    wq: tuple
    wk: tuple
    wv: tuple
    wo: tuple
    gate: tuple
    up: tuple
    down: tuple
    q_norm: Optional[np.ndarray] = None
    k_norm: Optional[np.ndarray] = None


@dataclass
class TokenRows:
    """``TokenOut::Rows { argmax, hidden }`` (gpu/types.rs:228-238): the greedy winner of every
    row and the output-normed hidden rows, what ``verify_tokens`` consumes (model/decode.rs:212-217)."""
    argmax: np.ndarray
    hidden: np.ndarray


@dataclass
class TokenReq:
    """gpu/types.rs:183-238, the fields the dequant-matvec path consumes."""
    layers: Sequence[TokenLayer]
    output_norm: np.ndarray
    output: tuple
    x: np.ndarray
    m: int
    rope: np.ndarray
    rot_dim: int
    eps: float
    hidden: int
    head_dim: int
    n_heads: int
    n_kv_heads: int
    argmax: bool = False
    attn_core: int = ATTN_IDENTITY
    kv: Optional["KvCache"] = None    # attn_core = ATTN_CAUSAL: the session's f16 KV cache (TokenReq.cache)
    pos: int = 0                      # cache position of row 0 (TokenReq.pos)
    scale: float = 0.0                # 1/sqrt(head_dim) (TokenReq.scale)
    embd: Optional[tuple] = None      # (ty, table bytes, vocab rows): TokenReq.embd
    token_id: Optional[int] = None    # with embd and m == 1: the input row is this token's embedding row


class KvCache:
    """The f16 KV cache of a session on the device (``KvCache``, crates/allpaka-model/src/kv.rs): per
    layer a K and a V slab of ``[capacity, kv_dim]`` halves.  Rows travel as uint16 (f16 bits)."""

    def __init__(self, gpu: "Gpu", n_layers: int, kv_dim: int, capacity: int):
        self._g = gpu
        h = C.c_void_p()
        rc = gpu._l.apk_kv_create(gpu._h, n_layers, kv_dim, capacity, C.byref(h))
        if rc != 0:
            raise GpuError(rc, gpu._err())
        self._h = h
        self.n_layers, self.kv_dim, self.capacity = n_layers, kv_dim, capacity

    def read(self, layer: int, pos0: int, n_pos: int):
        k = np.empty((n_pos, self.kv_dim), np.uint16)
        v = np.empty((n_pos, self.kv_dim), np.uint16)
        rc = self._g._l.apk_kv_read(self._g._h, self._h, layer, pos0, n_pos, k.ctypes.data, v.ctypes.data)
        if rc != 0:
            raise GpuError(rc, self._g._err())
        return k, v

    def write(self, layer: int, pos0: int, k, v) -> None:
        k = np.ascontiguousarray(k, dtype=np.uint16).reshape(-1, self.kv_dim)
        v = np.ascontiguousarray(v, dtype=np.uint16).reshape(-1, self.kv_dim)
        rc = self._g._l.apk_kv_write(self._g._h, self._h, layer, pos0, k.shape[0], k.ctypes.data, v.ctypes.data)
        if rc != 0:
            raise GpuError(rc, self._g._err())

    def close(self):
        if self._h and self._g._h:
            self._g._l.apk_kv_destroy(self._g._h, self._h)
        self._h = None


class Gpu:
    """One GPU context.  The module-level functions below forward to a
    process-wide instance, like the reference's lazily-initialised singleton
    (gpu/cuda/runtime/device.rs:267, 934-948)."""

    def __init__(self, device: int = -1):
        self._l = load_library()
        h = C.c_void_p()
        rc = self._l.apk_init(C.byref(h), device)
        if rc != 0:
            raise GpuError(rc, self._l.apk_last_error(None).decode())
        self._h = h
        self._attached = []   # keeps attached buffers alive
        self._token_cache = {}

    def close(self):
        if self._h:
            self._l.apk_shutdown(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- status handling ---------------------------------------------------
    def _err(self) -> str:
        return self._l.apk_last_error(self._h).decode(errors="replace")

    def _check(self, rc: int) -> bool:
        """True = executed, False = declined (caller returns None)."""
        if rc == 0:
            return True
        if rc > 0:
            self.last_decline = (rc, self._err())
            return False
        raise GpuError(rc, self._err())

    # -- gpu::attach / detach / is_attached (stub.rs:37-45) ------------------
    def attach(self, mapping: np.ndarray) -> bool:
        m = _u8(mapping)
        rc = self._l.apk_attach(self._h, m.ctypes.data, m.size)
        if rc == 0:
            self._attached.append(m)
        return self._check(rc)

    def detach(self, mapping: np.ndarray) -> None:
        m = _u8(mapping)
        self._check(self._l.apk_detach(self._h, m.ctypes.data, m.size))
        self._attached = [a for a in self._attached if a.ctypes.data != m.ctypes.data or a.size != m.size]
        self._token_cache.clear()

    def is_attached(self) -> bool:
        return bool(self._l.apk_is_attached(self._h))

    def register_matrix(self, w, ty: int, n_out: int, n_in: int) -> bool:
        w = _u8(w)
        return self._check(self._l.apk_register_matrix(self._h, w.ctypes.data, ty, n_out, n_in))

    # -- gpu::matvec (stub.rs:87-95) ----------------------------------------
    def matvec(self, ty: int, w, n_in: int, n_out: int, x, m: int = 1,
               act_mode: int = ACT_AUTO) -> Optional[np.ndarray]:
        w = _u8(w)
        x = _f32(x).reshape(-1)
        if x.size != m * n_in:
            raise ValueError(f"x has {x.size} values, expected {m} x {n_in}")
        y = np.empty((m, n_out), dtype=np.float32)
        rc = self._l.apk_matvec(self._h, w.ctypes.data, ty, n_in, n_out, x.ctypes.data, m, act_mode,
                                y.ctypes.data)
        return y if self._check(rc) else None

    # -- gpu::matvec_batch (stub.rs:97-99) ----------------------------------
    def matvec_batch(self, reqs: Sequence[MatvecReq], act_mode: int = ACT_Q8):
        if not reqs:
            return []
        arr = (_MatvecReq * len(reqs))()
        keep, ys = [], []
        for i, r in enumerate(reqs):
            w, x = _u8(r.w), _f32(r.x).reshape(-1)
            if x.size != r.m * r.n_in:
                raise ValueError(f"x has {x.size} values, expected {r.m} x {r.n_in}")
            # requests that share one activation array keep sharing it here
            for (ko, kx) in keep:
                if ko is r.x:
                    x = kx
            keep.append((r.x, x))
            y = np.empty((r.m, r.n_out), dtype=np.float32)
            ys.append(y)
            arr[i] = _MatvecReq(r.ty, w.ctypes.data, r.n_in, r.n_out, x.ctypes.data, r.m)
        yp = (C.c_void_p * len(reqs))(*[y.ctypes.data for y in ys])
        rc = self._l.apk_matvec_batch(self._h, C.addressof(arr), len(reqs), act_mode, C.addressof(yp))
        return ys if self._check(rc) else None

    # -- gpu::ffn_batch (stub.rs:101-103) -----------------------------------
    def ffn_batch(self, reqs: Sequence[FfnReq]):
        outs = []
        for r in reqs:
            x = _f32(r.x).reshape(-1)
            if x.size != r.m * r.hidden:
                return None  # the reference declines a mis-sized x (cuda/mod.rs:269-271)
            g, u, d = _u8(r.gate_w), _u8(r.up_w), _u8(r.down_w)
            req = _FfnReq(r.gate_ty, g.ctypes.data, r.up_ty, u.ctypes.data, r.down_ty, d.ctypes.data,
                          r.hidden, r.ffn, x.ctypes.data, r.m)
            y = np.empty((r.m, r.hidden), dtype=np.float32)
            if not self._check(self._l.apk_ffn(self._h, C.byref(req), y.ctypes.data)):
                return None
            outs.append(y)
        return outs

    # -- input half of gpu::attn_block (stub.rs:146-148) ---------------------
    def attn_in(self, ty, wq, wk, wv, hidden, head_dim, n_heads, n_kv_heads, x, m, gamma, eps, rope,
                rot_dim=None, q_norm=None, k_norm=None):
        wq, wk, wv = _u8(wq), _u8(wk), _u8(wv)
        x = _f32(x).reshape(-1)
        rope = _f32(rope).reshape(m, -1, 2)
        rot_dim = rope.shape[1] * 2 if rot_dim is None else rot_dim
        gamma = None if gamma is None else _f32(gamma)
        q_norm = None if q_norm is None else _f32(q_norm)
        k_norm = None if k_norm is None else _f32(k_norm)
        nq, nkv = n_heads * head_dim, n_kv_heads * head_dim
        q = np.empty((m, nq), np.float32)
        k = np.empty((m, nkv), np.float32)
        v = np.empty((m, nkv), np.float32)
        req = _AttnInReq(ty, wq.ctypes.data, wk.ctypes.data, wv.ctypes.data, hidden, head_dim, n_heads,
                         n_kv_heads, x.ctypes.data, m, _ptr(gamma), eps, _ptr(q_norm), _ptr(k_norm),
                         rope.ctypes.data, rot_dim)
        rc = self._l.apk_attn_in(self._h, C.byref(req), q.ctypes.data, k.ctypes.data, v.ctypes.data)
        return (q, k, v) if self._check(rc) else None

    # -- gpu::decode_token_checked / decode_token (stub.rs:150-161) ----------
    def _token_req(self, req: TokenReq):
        """Marshal once per distinct layer list; the C side keys its plan on the
        layer array's address, as the reference keys on borrowed slices."""
        key = id(req.layers)
        ent = self._token_cache.get(key)
        if ent is None:
            arr = (_TokenLayer * len(req.layers))()
            keep = []

            def mat(t):
                ty, w, n_out = t
                w = _u8(w)
                keep.append(w)
                return _Mat(ty, w.ctypes.data, n_out)

            def vec(a):
                if a is None:
                    return None
                a = _f32(a)
                keep.append(a)
                return a.ctypes.data

            for i, L in enumerate(req.layers):
                arr[i] = _TokenLayer(vec(L.attn_norm), vec(L.ffn_norm), mat(L.wq), mat(L.wk), mat(L.wv),
                                     mat(L.wo), vec(L.q_norm), vec(L.k_norm), mat(L.gate), mat(L.up),
                                     mat(L.down))
            on = _f32(req.output_norm)
            keep.append(on)
            ent = (arr, keep, on, mat(req.output), req.layers, mat)
            self._token_cache[key] = ent
        arr, keep, on, out_mat, _, mat = ent
        x = None if req.x is None else _f32(req.x).reshape(-1)
        rope = None if req.rope is None else _f32(req.rope).reshape(-1)
        embd = mat(req.embd) if req.embd is not None else _Mat(0, None, 0)
        use_token = req.embd is not None and req.token_id is not None
        creq = _TokenReq(C.addressof(arr), len(req.layers), on.ctypes.data, out_mat, _ptr(x), req.m,
                         _ptr(rope), req.rot_dim, req.eps, req.hidden, req.head_dim, req.n_heads,
                         req.n_kv_heads, req.attn_core, 1 if req.argmax else 0, embd,
                         int(req.token_id) if req.token_id is not None else 0, 1 if use_token else 0,
                         req.kv._h if req.kv is not None else None, int(req.pos), float(req.scale))
        return creq, (x, rope)

    def decode_token_checked(self, req: TokenReq, want_hidden: bool = False):
        """``TokenOut``: logits (argmax off), the winner ids (argmax on, m == 1), or
        :class:`TokenRows` (argmax on and m > 1, as the reference returns for a verify batch).
        With ``want_hidden`` the output-normed rows come along in every form: ``(result, hidden)``."""
        creq, keep = self._token_req(req)
        return self.decode_request(creq, want_hidden)

    def decode_request(self, creq: "_TokenReq", want_hidden: bool = False):
        """``apk_decode_token`` on a C request as it stands (e.g. a model's template with the input,
        rope rows, cache and position filled in)."""
        m, argmax = int(creq.m), bool(creq.argmax)
        rows = want_hidden or (argmax and m > 1)
        hidden = np.empty((m, int(creq.hidden)), dtype=np.float32) if rows else None
        if argmax:
            res = np.empty(m, dtype=np.uint32)
            out = _TokenOut(None, res.ctypes.data, _ptr(hidden))
        else:
            res = np.empty((m, int(creq.output.n_out)), dtype=np.float32)
            out = _TokenOut(res.ctypes.data, None, _ptr(hidden))
        rc = self._l.apk_decode_token(self._h, C.byref(creq), C.byref(out))
        if rc > 0:
            raise DecodeDecline(rc, self._err())
        if rc < 0:
            raise GpuError(rc, self._err())
        if argmax and m > 1:
            return TokenRows(res, hidden)
        return (res, hidden) if want_hidden else res

    def decode_token(self, req: TokenReq):
        try:
            return self.decode_token_checked(req)
        except DecodeDecline:
            return None

    def decode_greedy(self, req: TokenReq, n_tokens: int, rope_rows) -> Optional[np.ndarray]:
        """``decode_token`` with argmax followed by ``decode_greedy_continue`` (gpu/cuda/decode.rs:93-227):
        ``n_tokens`` greedy steps from ``req.token_id`` with one synchronisation; ``rope_rows`` holds one
        (sin, cos) row per step.  Returns the winners; None when declined."""
        creq, keep = self._token_req(req)
        rope = _f32(rope_rows).reshape(n_tokens, -1)
        out = np.empty(n_tokens, dtype=np.uint32)
        rc = self._l.apk_decode_greedy(self._h, C.byref(creq), n_tokens, rope.ctypes.data, out.ctypes.data)
        if rc > 0:
            self.last_decline = (rc, self._err())
            return None
        if rc < 0:
            raise GpuError(rc, self._err())
        return out

    def attend(self, kv: KvCache, layer: int, q, m: int, n_heads: int, pos: int, scale: float):
        """``gpu::attend_batch`` (AttnReq, gpu/types.rs:34-52): m query rows over one layer of the cache,
        row i over positions 0..=pos+i.  None when declined."""
        q = _f32(q).reshape(-1)
        out = np.empty((m, n_heads * 128), np.float32)
        rc = self._l.apk_attend(self._h, kv._h, layer, q.ctypes.data, m, n_heads, pos, scale, out.ctypes.data)
        return out if self._check(rc) else None

    def bench_attend(self, kv: KvCache, q, m: int, n_heads: int, pos: int, scale: float, reps: int = 10) -> float:
        """Microseconds per layer of the attention core, launched over every layer of ``kv`` in turn."""
        q = _f32(q).reshape(-1)
        us = C.c_float()
        rc = self._l.apk_bench_attend(self._h, kv._h, q.ctypes.data, m, n_heads, pos, scale, reps, C.byref(us))
        if rc != 0:
            raise GpuError(rc, self._err())
        return float(us.value)

    def decode_replay(self, req: TokenReq, iters: int) -> float:
        """Replay the token graph `iters` times on device-resident input; returns GPU ms."""
        creq, keep = self._token_req(req)
        ms = C.c_float()
        rc = self._l.apk_decode_replay(self._h, C.byref(creq), iters, C.byref(ms))
        if rc > 0:
            raise DecodeDecline(rc, self._err())
        if rc < 0:
            raise GpuError(rc, self._err())
        return ms.value

    # -- parity instrumentation ----------------------------------------------
    def debug_block_dots(self, ty, w, n_in, n_out, x, m=1):
        w, x = _u8(w), _f32(x).reshape(-1)
        dots = np.empty((m, n_out, n_in // 32), dtype=np.int32)
        rc = self._l.apk_debug_block_dots(self._h, w.ctypes.data, ty, n_in, n_out, x.ctypes.data, m,
                                          dots.ctypes.data)
        return dots if self._check(rc) else None

    def debug_q8_acts(self, x, gamma=None, eps=0.0):
        x = _f32(x).reshape(-1)
        gamma = None if gamma is None else _f32(gamma)
        d = np.empty(x.size // 32, np.float32)
        s = np.empty(x.size // 32, np.float32)
        q = np.empty(x.size, np.int8)
        rc = self._l.apk_debug_q8_acts(self._h, x.ctypes.data, x.size, _ptr(gamma), eps, d.ctypes.data,
                                       s.ctypes.data, q.ctypes.data)
        return (d, s, q) if self._check(rc) else None

    def debug_token_records(self, req: TokenReq, max_records: int = 512, dots_launch: int = -1,
                            dots_shape=None):
        """What every RMSNorm-fed matvec of one token worked on: a list of dicts with the residual
        rows ``x`` it normalised and the activation records ``d``, ``sum``, ``q`` it consumed
        (rows = tokens, or digit pairs in two-level mode), plus, for matvec launch number
        ``dots_launch``, its int32 block dots (``dots_shape`` = (rows, device rows, blocks))."""
        creq, keep = self._token_req(req)
        H, nb = req.hidden, req.hidden // 32
        x = np.zeros((max_records, MAX_M, H), np.float32)
        d = np.zeros((max_records, 16, nb), np.float32)
        s = np.zeros((max_records, 16, nb), np.float32)
        q = np.zeros((max_records, 16, H), np.int8)
        meta = np.zeros((max_records, 4), np.int32)
        n = C.c_uint32()
        dots = np.empty(dots_shape, np.int32) if dots_shape is not None else None
        rc = self._l.apk_debug_token_records(self._h, C.byref(creq), max_records, x.ctypes.data, d.ctypes.data,
                                             s.ctypes.data, q.ctypes.data, meta.ctypes.data, C.byref(n), dots_launch,
                                             _ptr(dots), 0 if dots is None else dots.size)
        if rc != 0:
            raise GpuError(rc, self._err())
        recs = []
        for i in range(n.value):
            rows, two, launch, ke = (int(v) for v in meta[i])
            recs.append({"x": x[i, :req.m], "d": d[i, :rows], "sum": s[i, :rows], "q": q[i, :rows],
                         "rows": rows, "two_level": bool(two), "launch": launch, "ke": ke})
        return (recs, dots) if dots is not None else recs

    def debug_set_wait_limit(self, cycles: int) -> None:
        """Cycle budget of the bounded device-side waits (0 = default)."""
        rc = self._l.apk_debug_set_wait_limit(self._h, cycles)
        if rc != 0:
            raise GpuError(rc, self._err())

    def debug_xch_timeout(self) -> int:
        """Run the exchange-collecting kernel against a peer that never delivers; returns the status."""
        return self._l.apk_debug_xch_timeout(self._h)

    def matvec_noalloc(self, ty: int, w, n_in: int, n_out: int, x_dev: int, m: int, y_dev: int,
                       stream: int = 0, act_mode: int = ACT_AUTO, wait: bool = True) -> bool:
        """apk_matvec_noalloc: for callers that may not allocate device memory here (VRAM fully
        budgeted, or a latency-bounded loop that cannot afford the stall).  `w` must already be resident;
        `x_dev`, `y_dev` and `stream` are raw device pointers / a cudaStream_t handle owned by the
        caller.  True = executed, False = declined (see ``last_decline``)."""
        w = _u8(w)
        rc = self._l.apk_matvec_noalloc(self._h, w.ctypes.data, ty, n_in, n_out, x_dev, m, act_mode, y_dev,
                                        stream, 1 if wait else 0)
        return self._check(rc)

    def debug_matvec_timeline(self, ty, w, n_in, n_out, x, m=1):
        """Per-CTA global-timer stamps (ns) of one matvec launch; see the C header."""
        w, x = _u8(w), _f32(x).reshape(-1)
        stamps = np.zeros((512, 8), dtype=np.uint64)
        n = C.c_uint32()
        rc = self._l.apk_debug_matvec_timeline(self._h, w.ctypes.data, ty, n_in, n_out, x.ctypes.data, m,
                                               stamps.ctypes.data, 512, C.byref(n))
        return stamps[: n.value] if self._check(rc) else None

    # -- benchmark utilities --------------------------------------------------
    def synth_matrix(self, w: np.ndarray, ty: int, n_out: int, n_in: int, seed: int,
                     write_host: bool = False) -> None:
        """Fill the matrix whose host bytes are `w` from the on-device generator."""
        rc = self._l.apk_debug_synth_matrix(self._h, w.ctypes.data, ty, n_out, n_in, seed,
                                            1 if write_host else 0)
        if rc != 0:
            raise GpuError(rc, self._err())

    def synth_release(self) -> None:
        rc = self._l.apk_debug_synth_release(self._h)
        if rc != 0:
            raise GpuError(rc, self._err())

    def bench_ring(self, op: str, copies: Sequence, reps: int = 20, act_mode: int = ACT_AUTO) -> float:
        """Microseconds per pass of one operator over a ring of distinct weight copies (device-resident
        inputs, launches chained back to back).  ``op`` = "matvec" (copies: MatvecReq), "attn_in"
        (copies: dicts with the arguments of :meth:`attn_in`) or "ffn" (copies: FfnReq)."""
        keep = []
        n = len(copies)
        br = _BenchReq(0, n, None, None, None, act_mode)
        if op == "matvec":
            arr = (_MatvecReq * n)()
            for i, r in enumerate(copies):
                w, x = _u8(r.w), _f32(r.x).reshape(-1)
                keep += [w, x]
                arr[i] = _MatvecReq(r.ty, w.ctypes.data, r.n_in, r.n_out, x.ctypes.data, r.m)
            br.op, br.mv = 0, C.addressof(arr)
        elif op == "attn_in":
            arr = (_AttnInReq * n)()
            for i, a in enumerate(copies):
                wq, wk, wv = _u8(a["wq"]), _u8(a["wk"]), _u8(a["wv"])
                x, rope = _f32(a["x"]).reshape(-1), _f32(a["rope"]).reshape(-1)
                gam = None if a.get("gamma") is None else _f32(a["gamma"])
                qn = None if a.get("q_norm") is None else _f32(a["q_norm"])
                kn = None if a.get("k_norm") is None else _f32(a["k_norm"])
                keep += [wq, wk, wv, x, rope, gam, qn, kn]
                arr[i] = _AttnInReq(a["ty"], wq.ctypes.data, wk.ctypes.data, wv.ctypes.data, a["hidden"], a["head_dim"],
                                    a["n_heads"], a["n_kv_heads"], x.ctypes.data, a["m"], _ptr(gam), a["eps"], _ptr(qn),
                                    _ptr(kn), rope.ctypes.data, a["rot_dim"])
            br.op, br.attn = 1, C.addressof(arr)
        elif op == "ffn":
            arr = (_FfnReq * n)()
            for i, r in enumerate(copies):
                g, u, d, x = _u8(r.gate_w), _u8(r.up_w), _u8(r.down_w), _f32(r.x).reshape(-1)
                keep += [g, u, d, x]
                arr[i] = _FfnReq(r.gate_ty, g.ctypes.data, r.up_ty, u.ctypes.data, r.down_ty, d.ctypes.data, r.hidden,
                                 r.ffn, x.ctypes.data, r.m)
            br.op, br.ffn = 2, C.addressof(arr)
        else:
            raise ValueError(op)
        us = C.c_float()
        rc = self._l.apk_bench_ring(self._h, C.byref(br), reps, C.byref(us))
        if rc != 0:
            raise GpuError(rc, self._err())
        return us.value

    def decode_profile(self, req: "TokenReq", reps: int = 1):
        """Per-launch GPU ms and algorithmic bytes of the five matvec kinds of a token."""
        creq, keep = self._token_req(req)
        ms = np.zeros(5, np.float32)
        by = np.zeros(5, np.float64)
        rc = self._l.apk_decode_profile(self._h, C.byref(creq), reps, ms.ctypes.data, by.ctypes.data)
        if rc != 0:
            raise GpuError(rc, self._err())
        names = ("qkv", "wo", "gate_up", "down", "lm_head")
        return {n: {"ms": float(t), "bytes": float(b)} for n, t, b in zip(names, ms, by)}

    def debug_token_timeline(self, req: "TokenReq", max_launches: int = 64):
        """Per-launch, per-CTA global-timer stamps (ns) of one un-graphed token; see the C header."""
        creq, keep = self._token_req(req)
        stamps = np.zeros((max_launches, 256, 8), dtype=np.uint64)
        nl, nc = C.c_uint32(), C.c_uint32()
        # the library writes [launch][n_ctas][8] densely; n_ctas is only known afterwards
        flat = stamps.reshape(-1)
        rc = self._l.apk_debug_token_timeline(self._h, C.byref(creq), flat.ctypes.data, max_launches,
                                              C.byref(nl), C.byref(nc))
        if rc != 0:
            raise GpuError(rc, self._err())
        return flat[: max_launches * nc.value * 8].reshape(max_launches, nc.value, 8)[: nl.value]

    # -- gpu::stats / decode_path_stats (common.rs:24-31, types.rs:271-278) --
    def stats_full(self) -> dict:
        st = _Stats()
        self._l.apk_stats(self._h, C.byref(st))
        return {n: getattr(st, n) for n, _ in _Stats._fields_}

    def stats(self):
        s = self.stats_full()
        return (s["calls"], s["launches"], s["encode_ns"], s["wait_ns"])

    def decode_path_stats(self):
        s = self.stats_full()
        return {"attempts": s["decode_attempts"], "successes": s["decode_successes"],
                "declines": s["decode_declines"]}

    # -- tensor parallel group -------------------------------------------------
    @staticmethod
    def dist_unique_id() -> bytes:
        l = load_library()
        buf = C.create_string_buffer(128)
        rc = l.apk_dist_unique_id(buf)
        if rc != 0:
            raise GpuError(rc, l.apk_last_error(None).decode())
        return buf.raw

    def p2p_export(self) -> bytes:
        """This rank's exchange-buffer handle (64 bytes) for the peer-memory reductions."""
        buf = C.create_string_buffer(64)
        rc = self._l.apk_dist_p2p_export(self._h, buf)
        if rc != 0:
            raise GpuError(rc, self._err())
        return buf.raw

    def p2p_open(self, handles: Sequence[bytes]) -> None:
        """Open every rank's handle (rank order); reductions then go over peer memory."""
        blob = C.create_string_buffer(b"".join(handles), 64 * len(handles))
        rc = self._l.apk_dist_p2p_open(self._h, blob)
        if rc != 0:
            raise GpuError(rc, self._err())

    def dist_set_exchange(self, peer_stores: bool) -> None:
        """Per-layer reductions through the peer-store exchange (True) or NCCL all-reduce (False)."""
        rc = self._l.apk_dist_set_exchange(self._h, 1 if peer_stores else 0)
        if rc != 0:
            raise GpuError(rc, self._err())

    def dist_init(self, rank: int, world: int, unique_id: bytes) -> None:
        buf = C.create_string_buffer(unique_id, 128)
        rc = self._l.apk_dist_init(self._h, rank, world, buf)
        if rc != 0:
            raise GpuError(rc, self._err())


SHARD_ROWS, SHARD_K = 1, 2


def shard_plan(kind: int, ty: int, n_out: int, n_in: int, rank: int, world: int, row_granule: int = 1):
    """(first row, rows, first column, columns) of the slice `rank` holds; None when
    the matrix does not divide.  Host arithmetic only: works without a GPU."""
    out = (C.c_uint32 * 4)()
    rc = load_library().apk_shard_plan(kind, ty, n_out, n_in, row_granule, rank, world, out)
    if rc > 0:
        return None
    if rc < 0:
        raise GpuError(rc, load_library().apk_last_error(None).decode())
    return tuple(int(v) for v in out)


# ---------------------------------------------------------------- module API
_GPU: Optional[Gpu] = None


def _gpu() -> Gpu:
    global _GPU
    if _GPU is None:
        _GPU = Gpu()
    return _GPU


def attach(mapping) -> bool:
    return _gpu().attach(mapping)


def detach(mapping) -> None:
    _gpu().detach(mapping)


def is_attached() -> bool:
    return _GPU is not None and _GPU.is_attached()


def matvec(ty, w, n_in, n_out, x):
    """gpu::matvec: one activation row, Q8 activations (m == 1)."""
    y = _gpu().matvec(ty, w, n_in, n_out, x, 1, ACT_AUTO)
    return None if y is None else y[0]


def matvec_batch(reqs, act_mode=ACT_Q8):
    return _gpu().matvec_batch(reqs, act_mode)


def ffn_batch(reqs):
    return _gpu().ffn_batch(reqs)


def decode_token_checked(req):
    return _gpu().decode_token_checked(req)


def decode_token(req):
    return _gpu().decode_token(req)


def stats():
    return _gpu().stats() if _GPU is not None else (0, 0, 0, 0)


def decode_path_stats():
    return _gpu().decode_path_stats()

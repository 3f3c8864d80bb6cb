"""GGUF model files: the reader and the dense-decoder model view of ``libapk_b200.so``
(``apk_gguf_*``, ``apk_model_*``), plus a small writer for synthetic files.

The reader mirrors ``GgufFile`` (crates/allpaka-gguf/src/tensors.rs:90-217, metadata.rs:194-297):
tensors are views into one read-only mapping of the file.  ``Model`` mirrors what ``Model::load``
binds for attention + dense-FFN decoders (crates/allpaka-model/src/model/loader.rs:100-260) and
``Config::from_gguf`` derives (crates/allpaka-model/src/config.rs:184-310)."""
from __future__ import annotations

import ctypes as C
import struct
from typing import Dict, Iterable, Optional, Sequence, Tuple

import numpy as np

from . import gpu as G

F32, F16 = 0, 1


class _Tensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("ty", C.c_uint32), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4),
                ("data", C.c_void_p), ("n_bytes", C.c_uint64)]


class _ModelInfo(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "rot_dim")] + \
               [("eps", C.c_float), ("rope_base", C.c_float), ("has_qk_norm", C.c_int), ("neox_reordered", C.c_int), ("tied", C.c_int)]


def _lib():
    l = G.load_library()
    if getattr(l, "_gguf_declared", False):
        return l
    l.apk_gguf_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    l.apk_gguf_close.argtypes = [C.c_void_p]
    l.apk_gguf_close.restype = None
    l.apk_gguf_n_tensors.argtypes = [C.c_void_p]
    l.apk_gguf_n_tensors.restype = C.c_uint64
    l.apk_gguf_tensor_at.argtypes = [C.c_void_p, C.c_uint64, C.POINTER(_Tensor)]
    l.apk_gguf_find.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(_Tensor)]
    l.apk_gguf_architecture.argtypes = [C.c_void_p]
    l.apk_gguf_architecture.restype = C.c_char_p
    l.apk_gguf_meta_u32.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint32)]
    l.apk_gguf_meta_f32.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_float)]
    l.apk_gguf_meta_str.argtypes = [C.c_void_p, C.c_char_p]
    l.apk_gguf_meta_str.restype = C.c_char_p
    l.apk_gguf_mapping.argtypes = [C.c_void_p, C.POINTER(C.c_uint64)]
    l.apk_gguf_mapping.restype = C.c_void_p
    l.apk_model_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    l.apk_model_get_info.argtypes = [C.c_void_p]
    l.apk_model_get_info.restype = C.POINTER(_ModelInfo)
    l.apk_model_token_req.argtypes = [C.c_void_p, C.c_void_p]
    l.apk_model_attach.argtypes = [C.c_void_p, C.c_void_p]
    l.apk_model_close.argtypes = [C.c_void_p]
    l.apk_model_close.restype = None
    l.apk_last_error.restype = C.c_char_p
    l._gguf_declared = True
    return l


class GgufError(Exception):
    def __init__(self, rc: int, msg: str):
        super().__init__(f"gguf error {rc}: {msg}")
        self.rc = rc


def _raise(l, rc):
    raise GgufError(rc, l.apk_last_error(None).decode(errors="replace"))


class GgufFile:
    """A parsed, mapped GGUF file.  Tensor data are numpy views into the mapping (no copy)."""

    def __init__(self, path: str):
        self._l = _lib()
        h = C.c_void_p()
        rc = self._l.apk_gguf_open(str(path).encode(), C.byref(h))
        if rc != 0:
            _raise(self._l, rc)
        self._h = h

    def close(self):
        if self._h:
            self._l.apk_gguf_close(self._h)
            self._h = None

    @property
    def architecture(self) -> str:
        return self._l.apk_gguf_architecture(self._h).decode()

    def _view(self, t: _Tensor):
        data = None
        if t.n_bytes:
            data = np.ctypeslib.as_array(C.cast(t.data, C.POINTER(C.c_uint8)), shape=(int(t.n_bytes),))
        return {"name": t.name.decode(), "ty": int(t.ty), "dims": [int(t.dims[i]) for i in range(t.n_dims)], "data": data}

    def tensors(self):
        t = _Tensor()
        out = []
        for i in range(self._l.apk_gguf_n_tensors(self._h)):
            self._l.apk_gguf_tensor_at(self._h, i, C.byref(t))
            out.append(self._view(t))
        return out

    def tensor(self, name: str) -> Optional[dict]:
        t = _Tensor()
        rc = self._l.apk_gguf_find(self._h, name.encode(), C.byref(t))
        return self._view(t) if rc == 0 else None

    def meta_u32(self, key: str) -> Optional[int]:
        v = C.c_uint32()
        return int(v.value) if self._l.apk_gguf_meta_u32(self._h, key.encode(), C.byref(v)) == 0 else None

    def meta_f32(self, key: str) -> Optional[float]:
        v = C.c_float()
        return float(v.value) if self._l.apk_gguf_meta_f32(self._h, key.encode(), C.byref(v)) == 0 else None

    def meta_str(self, key: str) -> Optional[str]:
        s = self._l.apk_gguf_meta_str(self._h, key.encode())
        return None if s is None else s.decode()

    def mapping(self) -> np.ndarray:
        n = C.c_uint64()
        p = self._l.apk_gguf_mapping(self._h, C.byref(n))
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(int(n.value),))


class Model:
    """The dense-decoder view of a file: configuration, checked tensors, a request template."""

    def __init__(self, f: GgufFile):
        self._l = _lib()
        self._f = f
        h = C.c_void_p()
        rc = self._l.apk_model_open(f._h, C.byref(h))
        if rc != 0:
            _raise(self._l, rc)
        self._h = h
        i = self._l.apk_model_get_info(h).contents
        self.info = {n: getattr(i, n) for n, _ in _ModelInfo._fields_}

    def attach(self, gpu: "G.Gpu") -> None:
        rc = self._l.apk_model_attach(gpu._h, self._h)
        if rc != 0:
            _raise(self._l, rc)

    def request(self) -> "G._TokenReq":
        """The C request over the model's tensors; fill x / token_id, rope, kv, pos before the call."""
        r = G._TokenReq()
        rc = self._l.apk_model_token_req(self._h, C.byref(r))
        if rc != 0:
            _raise(self._l, rc)
        return r

    def layer(self, i: int) -> "G._TokenLayer":
        r = self.request()
        return C.cast(r.layers, C.POINTER(G._TokenLayer))[i]

    def close(self):
        if self._h:
            self._l.apk_model_close(self._h)
            self._h = None


# ------------------------------------------------------------------ writer (synthetic files)

def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def write_file(path: str, meta: Dict[str, object], tensors: Sequence[Tuple[str, int, Sequence[int], np.ndarray]],
               alignment: int = 32, version: int = 3) -> None:
    """Write a GGUF file: ``meta`` values are str, int (u32), float (f32), bool or a list of ints
    (u32 array) / strs (string array); ``tensors`` are (name, ggml type, dims, raw bytes)."""
    out = bytearray(b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(meta) + (1 if alignment != 32 else 0)))
    if alignment != 32:
        out += _s(b"general.alignment") + struct.pack("<II", 4, alignment)
    for k, v in meta.items():
        out += _s(k.encode())
        if isinstance(v, bool):
            out += struct.pack("<IB", 7, int(v))
        elif isinstance(v, str):
            out += struct.pack("<I", 8) + _s(v.encode())
        elif isinstance(v, int):
            out += struct.pack("<II", 4, v)
        elif isinstance(v, float):
            out += struct.pack("<If", 6, v)
        elif isinstance(v, (list, tuple)) and all(isinstance(e, str) for e in v):
            out += struct.pack("<IIQ", 9, 8, len(v)) + b"".join(_s(e.encode()) for e in v)
        elif isinstance(v, (list, tuple)):
            out += struct.pack("<IIQ", 9, 4, len(v)) + b"".join(struct.pack("<I", e) for e in v)
        else:
            raise TypeError(f"metadata value of {k}")
    offs, pos = [], 0
    for _, _, _, data in tensors:
        offs.append(pos)
        pos += (len(np.asarray(data).reshape(-1).view(np.uint8)) + alignment - 1) // alignment * alignment
    for (name, ty, dims, _), off in zip(tensors, offs):
        out += _s(name.encode()) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", ty, off)
    out += bytes(-len(out) % alignment)
    with open(path, "wb") as fh:
        fh.write(out)
        for (_, _, _, data), off in zip(tensors, offs):
            b = np.ascontiguousarray(data).reshape(-1).view(np.uint8).tobytes()
            fh.write(b + bytes(-len(b) % alignment))

"""Python view of the GGUF header parser (``mg_gguf_*`` in the C ABI): the reference's
``GgufFile`` (crates/modgrad-device/src/kfd/gguf.rs:98-234).  Needs no GPU."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from .backend import Runtime

# ggml type ids (gguf.rs:13-31)
F32, F16, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 12, 13, 14, 30


@dataclass
class TensorInfo:
    name: str
    dims: tuple
    dtype: int
    file_offset: int
    data_bytes: int


class GgufFile:
    def __init__(self, handle: int, keep=None):
        self.handle = handle
        self._keep = keep  # the buffer behind parse_memory
        self._lib = _lib.load()

    @classmethod
    def open(cls, path) -> "GgufFile":
        lib = _lib.load()
        h = C.c_void_p()
        if lib.mg_gguf_open(str(path).encode(), C.byref(h)) != 0:
            raise Runtime(lib.mg_gguf_last_error().decode())
        return cls(h.value)

    @classmethod
    def parse(cls, data: bytes) -> "GgufFile":
        lib = _lib.load()
        buf = np.frombuffer(data, dtype=np.uint8).copy()
        h = C.c_void_p()
        if lib.mg_gguf_parse_memory(buf.ctypes.data_as(C.c_void_p), buf.size, C.byref(h)) != 0:
            raise Runtime(lib.mg_gguf_last_error().decode())
        return cls(h.value, keep=buf)

    def close(self):
        if self.handle:
            self._lib.mg_gguf_close(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def version(self) -> int:
        return self._lib.mg_gguf_version(self.handle)

    @property
    def data_offset(self) -> int:
        return self._lib.mg_gguf_data_offset(self.handle)

    def tensors(self) -> list[TensorInfo]:
        out = []
        for i in range(self._lib.mg_gguf_n_tensors(self.handle)):
            name, nd, dt = C.c_char_p(), C.c_int(), C.c_uint32()
            dims = (C.c_uint64 * 4)()
            off, nb = C.c_uint64(), C.c_uint64()
            self._lib.mg_gguf_tensor(self.handle, i, C.byref(name), C.byref(nd), dims, C.byref(dt), C.byref(off), C.byref(nb))
            out.append(TensorInfo(name.value.decode(), tuple(int(d) for d in dims[:min(nd.value, 4)]), dt.value,
                                  off.value, nb.value))
        return out

    def meta_u32(self, key: str):
        v = C.c_uint32()
        return v.value if self._lib.mg_gguf_meta_u32(self.handle, key.encode(), C.byref(v)) == 0 else None

    def meta_f32(self, key: str):
        v = C.c_float()
        return v.value if self._lib.mg_gguf_meta_f32(self.handle, key.encode(), C.byref(v)) == 0 else None

    def meta_str(self, key: str):
        s = self._lib.mg_gguf_meta_str(self.handle, key.encode())
        return s.decode() if s is not None else None

    def meta_array_len(self, key: str) -> int:
        return int(self._lib.mg_gguf_meta_array_len(self.handle, key.encode()))

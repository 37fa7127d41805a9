"""Python view of the Q4_K residency container (``mg_linear_q4k_*``): the reference's
``LinearResidentQuantized`` (crates/modgrad-compute/src/neuron.rs:866-1250)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .backend import DeviceBuffer, Runtime, cuda_check


def quantize_row_q4_k(x: np.ndarray) -> np.ndarray:
    """Host quantiser, canonical element order; x.size % 256 == 0."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    out = np.empty(x.size // 256 * 144, dtype=np.uint8)
    if _lib.load().mg_quantize_row_q4_k(x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), x.size) != 0:
        raise Runtime("quantize_row_q4_k: length must be a positive multiple of 256")
    return out


class LinearResidentQuantized:
    def __init__(self, handle: int, in_dim: int, out_dim: int):
        self._lib, self._h, self.in_dim, self.out_dim = _lib.load(), handle, in_dim, out_dim

    @classmethod
    def from_linear(cls, weight: np.ndarray, bias: np.ndarray | None = None) -> "LinearResidentQuantized":
        """weight: fp32 [out_dim][in_dim]; quantised on the host, nothing allocated on the device."""
        w = np.ascontiguousarray(weight, dtype=np.float32)
        out_dim, in_dim = w.shape
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        h = C.c_void_p()
        rc = _lib.load().mg_linear_q4k_from_f32(w.ctypes.data_as(C.c_void_p), None if b is None else b.ctypes.data_as(C.c_void_p),
                                                in_dim, out_dim, C.byref(h))
        if rc != 0:
            raise Runtime("LinearResidentQuantized.from_linear: weight rows must be a multiple of 256 long")
        return cls(h.value, in_dim, out_dim)

    @classmethod
    def from_blocks(cls, q4k: np.ndarray, in_dim: int, out_dim: int, bias: np.ndarray | None = None):
        q = np.ascontiguousarray(q4k, dtype=np.uint8).reshape(-1)
        if q.size != out_dim * (in_dim // 256) * 144:
            raise Runtime("from_blocks: byte count does not match the shape")
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        h = C.c_void_p()
        rc = _lib.load().mg_linear_q4k_from_blocks(q.ctypes.data_as(C.c_void_p), None if b is None else b.ctypes.data_as(C.c_void_p),
                                                   in_dim, out_dim, C.byref(h))
        if rc != 0:
            raise Runtime("LinearResidentQuantized.from_blocks: bad shape")
        return cls(h.value, in_dim, out_dim)

    def close(self):
        if getattr(self, "_h", None):
            self._lib.mg_linear_q4k_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_expanded(self, expanded: bool):
        self._lib.mg_linear_q4k_set_expanded(self._h, int(expanded))

    def is_resident(self) -> bool:
        return bool(self._lib.mg_linear_q4k_is_resident(self._h))

    def host_size_bytes(self) -> int:
        return int(self._lib.mg_linear_q4k_host_size_bytes(self._h))

    def device_size_bytes(self) -> int:
        return int(self._lib.mg_linear_q4k_device_size_bytes(self._h))

    def host_blocks(self) -> np.ndarray:
        n = C.c_size_t()
        p = self._lib.mg_linear_q4k_host_blocks(self._h, C.byref(n))
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(n.value,)).copy()

    def ensure_resident(self):
        cuda_check(self._lib.mg_linear_q4k_ensure_resident(self._h, None), "ensure_resident")

    def evict(self):
        self._lib.mg_linear_q4k_evict(self._h)

    def forward(self, x_dev: DeviceBuffer, out_dev: DeviceBuffer, auto_evict: bool = False):
        cuda_check(self._lib.mg_linear_q4k_forward(self._h, x_dev.ptr, out_dev.ptr, int(auto_evict), None), "forward")

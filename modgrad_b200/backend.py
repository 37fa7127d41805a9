"""Python view of the host-side mirror of modgrad's operator surface for the Q4_K path.

Thin wrappers over the C ABI (include/modgrad_cuda.h); names and argument meaning follow
the reference:

* ``QuantKind``, ``Matvec``, ``DequantQ4KResident``  crates/modgrad-device/src/backend/op.rs:22-29, :178-186, :479-483
* ``BackendError`` and its kinds                     backend/mod.rs:109-123
* ``CudaBackend.{name,supports,dispatch,invalidate_cache}``  backend/mod.rs:148-176
* ``ops.matvec`` / ``ops.dequant_q4k_resident``      backend/ops.rs:82-90, :531-539
* ``DeviceBuffer`` (``HipBuffer``)                   backend/rocm.rs:603-738
* ``kern.*`` no-sync launch wrappers                 backend/rocm.rs:943-1078
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

import numpy as np

from . import _lib

BLOCK_BYTES = 144
BLOCK_ELEMS = 256


class QuantKind(enum.IntEnum):
    F32 = 0
    Q4K = 1


class BackendError(RuntimeError):
    """Base of the four reference error kinds."""


class Unsupported(BackendError):
    pass


class OutOfMemory(BackendError):
    pass


class DeviceLost(BackendError):
    pass


class Runtime(BackendError):
    pass


_KINDS = {-1: Unsupported, -2: OutOfMemory, -3: DeviceLost, -4: Runtime}


def cuda_check(code: int, what: str) -> None:
    """Non-zero launcher code -> ``Runtime(f"{what}: {error string}")`` (rocm.rs:947-949)."""
    if code != 0:
        msg = _lib.load().mg_get_error_string(code).decode()
        if code == 2:
            raise OutOfMemory("out of device memory")
        raise Runtime(f"{what}: {msg}")


def _np_ptr(a: np.ndarray) -> C.c_void_p:
    return a.ctypes.data_as(C.c_void_p)


@dataclass
class Matvec:
    """``Op::Matvec``: out = weight @ x + bias, host slices; weight is opaque bytes for Q4K."""
    x: np.ndarray
    weight: np.ndarray
    bias: np.ndarray
    out: np.ndarray
    out_dim: int
    in_dim: int
    quant: QuantKind


@dataclass
class DequantQ4KResident:
    """``Op::DequantQ4KResident``: device pointers (ints), ``n_blocks`` super-blocks."""
    q4k_dev: int
    fp32_dev: int
    n_blocks: int


class DeviceBuffer:
    """Owning device allocation, the counterpart of ``HipBuffer``."""

    def __init__(self, nbytes: int):
        self._lib = _lib.load()
        p = C.c_void_p()
        cuda_check(self._lib.mg_malloc(C.byref(p), max(1, nbytes)), "cudaMalloc")
        self.ptr = p.value
        self.bytes = nbytes

    def free(self):
        if getattr(self, "ptr", None):
            self._lib.mg_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def copy_from_host_bytes(self, src) -> None:
        a = np.ascontiguousarray(src).view(np.uint8).reshape(-1)
        if a.size > self.bytes:
            raise Runtime(f"copy_from_host_bytes: src {a.size} > buf {self.bytes}")
        cuda_check(self._lib.mg_memcpy_h2d(self.ptr, _np_ptr(a), a.size), "cudaMemcpy H2D bytes")

    def copy_from_host(self, src) -> None:
        self.copy_from_host_bytes(np.ascontiguousarray(src, dtype=np.float32))

    def copy_to_host(self, n_f32: int) -> np.ndarray:
        out = np.empty(n_f32, dtype=np.float32)
        if n_f32 * 4 > self.bytes:
            raise Runtime(f"copy_to_host: dst {n_f32 * 4} > buf {self.bytes}")
        cuda_check(self._lib.mg_memcpy_d2h(_np_ptr(out), self.ptr, n_f32 * 4), "cudaMemcpy D2H")
        return out

    def copy_to_host_bytes(self, dst: np.ndarray) -> np.ndarray:
        """Raw bytes back to a contiguous host array (any dtype)."""
        n = dst.nbytes
        if n > self.bytes or not dst.flags["C_CONTIGUOUS"]:
            raise Runtime(f"copy_to_host_bytes: dst {n} > buf {self.bytes} or not contiguous")
        cuda_check(self._lib.mg_memcpy_d2h(_np_ptr(dst), self.ptr, n), "cudaMemcpy D2H bytes")
        return dst

    def u8_at(self, offset: int) -> int:
        return self.ptr + offset

    def matvec_q4k(self, x, out_dim: int, blocks_per_row: int, out: np.ndarray | None = None) -> np.ndarray:
        """Resident weight, host x in, host y out (``HipBuffer::matvec_q4k``)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.size < blocks_per_row * BLOCK_ELEMS:
            raise Runtime("matvec_q4k: x shorter than blocks_per_row*256")
        y = out if out is not None else np.empty(out_dim, dtype=np.float32)
        cuda_check(self._lib.mg_buffer_matvec_q4k(self.ptr, self.bytes, _np_ptr(x), _np_ptr(y), out_dim,
                                                  blocks_per_row), "launch_matvec_q4k")
        return y

    def matvec_q4k_into(self, x_dev: "DeviceBuffer", y_dev: "DeviceBuffer", out_dim: int, blocks_per_row: int) -> None:
        """Device x / y, synchronises (``HipBuffer::matvec_q4k_into``)."""
        cuda_check(self._lib.mg_buffer_matvec_q4k_into(self.ptr, x_dev.ptr, y_dev.ptr, out_dim, blocks_per_row),
                   "launch_matvec_q4k")


class kern:
    """Raw no-sync launch wrappers over device pointers (ints); one ``sync`` per token."""

    @staticmethod
    def sync() -> None:
        cuda_check(_lib.load().mg_device_synchronize(), "cudaDeviceSynchronize")

    @staticmethod
    def vram_free_total() -> tuple[int, int]:
        f, t = C.c_size_t(), C.c_size_t()
        cuda_check(_lib.load().mg_mem_get_info(C.byref(f), C.byref(t)), "cudaMemGetInfo")
        return f.value, t.value

    @staticmethod
    def matvec_q4k(w: int, x: int, y: int, out_dim: int, bpr: int, stream: int | None = None) -> None:
        L = _lib.load()
        code = (L.launch_matvec_q4k(w, x, y, out_dim, bpr) if stream is None
                else L.launch_matvec_q4k_on_stream(w, x, y, out_dim, bpr, stream))
        cuda_check(code, "matvec_q4k")

    @staticmethod
    def quantize_q8_1(x: int, xq: int, xd: int, xsum: int, n: int, stream: int | None = None) -> None:
        """``kern::quantize_q8_1`` (rocm.rs:971): f32 x -> int8 + per-32 scale + per-32 sum."""
        L = _lib.load()
        code = (L.launch_quantize_q8_1(x, xq, xd, xsum, n) if stream is None
                else L.launch_quantize_q8_1_on_stream(x, xq, xd, xsum, n, stream))
        cuda_check(code, "quantize_q8_1")

    @staticmethod
    def matvec_q4k_dp4a(w: int, xq: int, xd: int, xsum: int, y: int, out_dim: int, bpr: int,
                        stream: int | None = None) -> None:
        """``kern::matvec_q4k_dp4a`` (rocm.rs:973-975): the lossy int8-activation matvec."""
        L = _lib.load()
        code = (L.launch_matvec_q4k_dp4a(w, xq, xd, xsum, y, out_dim, bpr) if stream is None
                else L.launch_matvec_q4k_dp4a_on_stream(w, xq, xd, xsum, y, out_dim, bpr, stream))
        cuda_check(code, "matvec_q4k_dp4a")

    @staticmethod
    def dequant_q4k(q4k: int, n_blocks: int, out: int, stream: int | None = None) -> None:
        L = _lib.load()
        code = (L.launch_dequant_q4k(q4k, n_blocks, out) if stream is None
                else L.launch_dequant_q4k_on_stream(q4k, n_blocks, out, stream))
        cuda_check(code, "dequant_q4k")


class CudaBackend:
    """The CUDA ``Backend``: claims ``Matvec{quant: Q4K}`` and ``DequantQ4KResident``."""

    def __init__(self, handle: int):
        self._lib = _lib.load()
        self._h = handle

    @classmethod
    def try_new(cls, device: int = 0) -> "CudaBackend | None":
        """``None`` when no CUDA device answers (the reference's ``try_new() -> Option``)."""
        h = C.c_void_p()
        if _lib.load().mg_backend_create(device, C.byref(h)) != 0 or not h.value:
            return None
        return cls(h.value)

    def close(self):
        if self._h:
            self._lib.mg_backend_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def name(self) -> str:
        return self._lib.mg_backend_name(self._h).decode()

    def device_info(self) -> str:
        return self._lib.mg_backend_device_info(self._h).decode()

    def _matvec_args(self, op: Matvec):
        w = op.weight.view(np.uint8).reshape(-1) if isinstance(op.weight, np.ndarray) else op.weight
        bias = op.bias if op.bias is not None else np.empty(0, dtype=np.float32)
        return (self._h, _np_ptr(op.x), op.x.size, _np_ptr(w), w.size, _np_ptr(bias), bias.size,
                _np_ptr(op.out), op.out.size, op.out_dim, op.in_dim, int(op.quant))

    def supports(self, op) -> bool:
        if isinstance(op, Matvec):
            return bool(self._lib.mg_backend_supports_matvec(*self._matvec_args(op)))
        if isinstance(op, DequantQ4KResident):
            return bool(self._lib.mg_backend_supports_dequant_q4k_resident(self._h, op.q4k_dev, op.fp32_dev, op.n_blocks))
        return False

    def dispatch(self, op) -> None:
        if isinstance(op, Matvec):
            code = self._lib.mg_backend_dispatch_matvec(*self._matvec_args(op))
        elif isinstance(op, DequantQ4KResident):
            code = self._lib.mg_backend_dispatch_dequant_q4k_resident(self._h, op.q4k_dev, op.fp32_dev, op.n_blocks)
        else:
            raise Unsupported(f"backend 'cuda' does not support op '{type(op).__name__}'")
        if code != 0:
            raise _KINDS.get(code, Runtime)(self._lib.mg_backend_last_error(self._h).decode())

    def invalidate_cache(self) -> None:
        self._lib.mg_backend_invalidate_cache(self._h)

    def cached_weights(self) -> int:
        return int(self._lib.mg_backend_cached_weights(self._h))


_registry: CudaBackend | None = None


def registry() -> CudaBackend:
    """The single-backend registry: CUDA or an error — no CPU arm, no fall-through."""
    global _registry
    if _registry is None:
        _registry = CudaBackend.try_new(0)
        if _registry is None:
            raise Unsupported("backend '<none>': no CUDA device (there is no CPU fallback for Q4_K)")
    return _registry


class ops:
    """Facade functions with the reference's signatures (backend/ops.rs)."""

    @staticmethod
    def matvec(x, weight, bias, out, out_dim: int, in_dim: int, quant: QuantKind) -> None:
        registry().dispatch(Matvec(x, weight, bias, out, out_dim, in_dim, quant))

    @staticmethod
    def dequant_q4k_resident(q4k_dev: int, fp32_dev: int, n_blocks: int) -> None:
        registry().dispatch(DequantQ4KResident(q4k_dev, fp32_dev, n_blocks))

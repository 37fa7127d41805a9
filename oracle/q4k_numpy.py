"""Independent numpy restatement of the Q4_K format functions.  TEST INFRASTRUCTURE ONLY.

Written from the format description (not from q4k_oracle.c) so that the two can be
checked against each other:

* ``f16_to_f32``          crates/modgrad-device/src/kfd/gguf.rs:281-292
* ``scale_min_k4``        gguf.rs:334-342
* ``pack_scales_mins``    gguf.rs:349-358
* ``dequantize``          gguf.rs:364-404 (ggml element order; two f32 roundings per weight)
* ``matvec_f64``          dequantised weights times x with f64 accumulation
                          (crates/modgrad-device/examples/rocm_matvec_check.rs:38-47)

PARITY UNPINNED: the reference (Rust) could not be run where this was written and has no
Q4_K golden vectors; see tests/golden/ for the hand-built known-answer blocks.
"""
from __future__ import annotations

import numpy as np

BLOCK_BYTES = 144
BLOCK_ELEMS = 256


def f16_to_f32(h: np.ndarray) -> np.ndarray:
    """Half bits -> f32.  Exponent 31 (inf and NaN) maps to NaN as in the reference."""
    h = np.asarray(h, dtype=np.uint16)
    out = h.view(np.float16).astype(np.float32)  # exact for every finite half, incl. sub-normals
    out = np.where(((h >> 10) & 0x1F) == 31, np.float32(np.nan), out)
    return out.astype(np.float32)


def scale_min_k4(scales: np.ndarray):
    """scales: (..., 12) uint8 -> (sc, m) each (..., 8) uint8."""
    s = np.asarray(scales, dtype=np.uint8)
    sc = np.empty(s.shape[:-1] + (8,), dtype=np.uint8)
    m = np.empty_like(sc)
    sc[..., :4] = s[..., 0:4] & 63
    m[..., :4] = s[..., 4:8] & 63
    sc[..., 4:] = (s[..., 8:12] & 0x0F) | ((s[..., 0:4] >> 6) << 4)
    m[..., 4:] = (s[..., 8:12] >> 4) | ((s[..., 4:8] >> 6) << 4)
    return sc, m


def pack_scales_mins(sc: np.ndarray, m: np.ndarray) -> np.ndarray:
    """(…, 8) six-bit scales and mins -> (…, 12) packed header bytes."""
    sc = np.asarray(sc, dtype=np.uint8)
    m = np.asarray(m, dtype=np.uint8)
    out = np.empty(sc.shape[:-1] + (12,), dtype=np.uint8)
    out[..., 0:4] = (sc[..., 0:4] & 0x3F) | (((sc[..., 4:8] >> 4) & 3) << 6)
    out[..., 4:8] = (m[..., 0:4] & 0x3F) | (((m[..., 4:8] >> 4) & 3) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 0x0F) | ((m[..., 4:8] & 0x0F) << 4)
    return out


def dequantize(blocks: np.ndarray) -> np.ndarray:
    """(n,144) uint8 -> (n,256) f32 in ggml order, bit-exact to the scalar specification."""
    b = np.asarray(blocks, dtype=np.uint8).reshape(-1, BLOCK_BYTES)
    n = b.shape[0]
    d = f16_to_f32(b[:, 0:2].copy().view(np.uint16)[:, 0])
    dmin = f16_to_f32(b[:, 2:4].copy().view(np.uint16)[:, 0])
    d = np.where(np.isfinite(d), d, np.float32(0)).astype(np.float32)
    dmin = np.where(np.isfinite(dmin), dmin, np.float32(0)).astype(np.float32)
    sc, m = scale_min_k4(b[:, 4:16])
    dsc = (d[:, None] * sc.astype(np.float32)).astype(np.float32)       # fl(d*sc)   (n,8)
    dm = (dmin[:, None] * m.astype(np.float32)).astype(np.float32)      # fl(dmin*m) (n,8)
    qs = b[:, 16:144].reshape(n, 4, 32)
    q = np.empty((n, 4, 2, 32), dtype=np.float32)
    q[:, :, 0, :] = (qs & 0x0F).astype(np.float32)
    q[:, :, 1, :] = (qs >> 4).astype(np.float32)
    q = q.reshape(n, 8, 32)
    prod = (dsc[:, :, None] * q).astype(np.float32)                      # fl(fl(d*sc)*q)
    w = (prod - dm[:, :, None]).astype(np.float32)
    return w.reshape(n, BLOCK_ELEMS)


def matvec_f64(w_blocks: np.ndarray, x: np.ndarray, out_dim: int, bpr: int) -> np.ndarray:
    w = dequantize(w_blocks).reshape(out_dim, bpr * BLOCK_ELEMS).astype(np.float64)
    return w @ np.asarray(x, dtype=np.float32)[: bpr * BLOCK_ELEMS].astype(np.float64)


# ---- Q5_K / Q6_K (independent restatements, vectorised differently from the C oracle) ------------
def half_bits_to_f32_zero_nonfinite(h: np.ndarray) -> np.ndarray:
    v = f16_to_f32(h)
    return np.where(np.isfinite(v), v, np.float32(0)).astype(np.float32)


def unpack_scales_mins(scales: np.ndarray):
    return scale_min_k4(scales)


def dequantize_q5k(blocks: np.ndarray) -> np.ndarray:
    """crates/modgrad-device/src/kfd/gguf.rs:421-455, all blocks at once."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 176)
    n = b.shape[0]
    d = half_bits_to_f32_zero_nonfinite(b[:, 0:2].copy().view(np.uint16).reshape(n))
    dmin = half_bits_to_f32_zero_nonfinite(b[:, 2:4].copy().view(np.uint16).reshape(n))
    sc, m = unpack_scales_mins(b[:, 4:16])
    qh, ql = b[:, 16:48], b[:, 48:176].reshape(n, 4, 32)
    out = np.empty((n, 8, 32), dtype=np.float32)
    for g in range(4):
        for hi in range(2):
            s = 2 * g + hi
            nib = (ql[:, g] >> 4) if hi else (ql[:, g] & 0xF)
            hbit = ((qh >> s) & 1).astype(np.uint8) * 16
            q = (nib + hbit).astype(np.float32)
            d1 = (d * sc[:, s].astype(np.float32)).astype(np.float32)
            m1 = (dmin * m[:, s].astype(np.float32)).astype(np.float32)
            out[:, s] = ((d1[:, None] * q).astype(np.float32) - m1[:, None]).astype(np.float32)
    return out.reshape(-1)


def dequantize_q6k(blocks: np.ndarray) -> np.ndarray:
    """crates/modgrad-device/src/kfd/gguf.rs:458-484, all blocks at once."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 210)
    n = b.shape[0]
    ql, qh = b[:, 0:128].reshape(n, 2, 64), b[:, 128:192].reshape(n, 2, 32)
    sc = b[:, 192:208].copy().view(np.int8).reshape(n, 2, 8).astype(np.float32)
    d = half_bits_to_f32_zero_nonfinite(b[:, 208:210].copy().view(np.uint16).reshape(n))
    out = np.empty((n, 2, 4, 32), dtype=np.float32)
    for k in range(4):  # q1..q4: low/high nibble of ql[l] / ql[l+32], two bits of qh at 2k
        src = ql[:, :, (k & 1) * 32:(k & 1) * 32 + 32]
        nib = (src >> 4) if k >= 2 else (src & 0xF)
        q = (nib.astype(np.int32) | (((qh >> (2 * k)) & 3).astype(np.int32) << 4)) - 32
        s = np.stack([sc[:, :, 2 * k], sc[:, :, 2 * k + 1]], axis=-1)        # scale of l < 16, l >= 16
        s = np.repeat(s, 16, axis=-1)                                         # (n, 2, 32)
        ds = (d[:, None, None] * s).astype(np.float32)
        out[:, :, k] = (ds * q.astype(np.float32)).astype(np.float32)
    return out.reshape(-1)

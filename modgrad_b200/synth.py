"""Seeded synthetic Q4_K inputs (the stand-in for GGUF checkpoints, which are not available).

Every consumer — the CUDA path, the CPU oracle in the tests, the CPU baseline in the
benchmark — receives the SAME host bytes produced here and uploaded verbatim; nothing is
generated separately per side.  Distributions (per 144-byte super-block):

* ``d``, ``dmin``: half( |N(0,1)| * 0.01 )
* 8 six-bit scales and 8 six-bit mins: uniform integers in [0, 63], packed in the GGUF
  12-byte layout (crates/modgrad-device/src/kfd/gguf.rs:349-358)
* 128 quant bytes: uniform in [0, 255]  (each nibble uniform in [0, 15])

PRNG: ``numpy.random.Generator(numpy.random.PCG64(seed))``; draw order per call is
(d,dmin) normals -> scales -> mins -> quant bytes, each for all blocks at once.
"""
from __future__ import annotations

import numpy as np

BLOCK_BYTES = 144
BLOCK_ELEMS = 256


def pack_scales_mins(sc: np.ndarray, m: np.ndarray) -> np.ndarray:
    """(n,8) six-bit scales / mins -> (n,12) header bytes (gguf.rs:349-358)."""
    sc = sc.astype(np.uint8)
    m = m.astype(np.uint8)
    out = np.empty(sc.shape[:-1] + (12,), dtype=np.uint8)
    out[..., 0:4] = (sc[..., 0:4] & 0x3F) | (((sc[..., 4:8] >> 4) & 3) << 6)
    out[..., 4:8] = (m[..., 0:4] & 0x3F) | (((m[..., 4:8] >> 4) & 3) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 0x0F) | ((m[..., 4:8] & 0x0F) << 4)
    return out


def q4k_blocks(n_blocks: int, rng: np.random.Generator) -> np.ndarray:
    """``n_blocks`` random super-blocks as an (n_blocks, 144) uint8 array."""
    out = np.empty((n_blocks, BLOCK_BYTES), dtype=np.uint8)
    dd = (np.abs(rng.standard_normal((n_blocks, 2), dtype=np.float32)) * np.float32(0.01)).astype(np.float16)
    out[:, 0:4] = dd.view(np.uint8).reshape(n_blocks, 4)
    sc = rng.integers(0, 64, size=(n_blocks, 8), dtype=np.uint8)
    m = rng.integers(0, 64, size=(n_blocks, 8), dtype=np.uint8)
    out[:, 4:16] = pack_scales_mins(sc, m)
    out[:, 16:144] = rng.integers(0, 256, size=(n_blocks, 128), dtype=np.uint8)
    return out


def q5k_blocks(n_blocks: int, rng: np.random.Generator) -> np.ndarray:
    """Random Q5_K super-blocks (176 bytes: d, dmin, scales[12], qh[32], ql[128];
    crates/modgrad-device/src/kfd/gguf.rs:421-432), same distributions as the Q4_K generator."""
    out = np.empty((n_blocks, 176), dtype=np.uint8)
    dd = (np.abs(rng.standard_normal((n_blocks, 2), dtype=np.float32)) * np.float32(0.01)).astype(np.float16)
    out[:, 0:4] = dd.view(np.uint8).reshape(n_blocks, 4)
    sc = rng.integers(0, 64, size=(n_blocks, 8), dtype=np.uint8)
    m = rng.integers(0, 64, size=(n_blocks, 8), dtype=np.uint8)
    out[:, 4:16] = pack_scales_mins(sc, m)
    out[:, 16:176] = rng.integers(0, 256, size=(n_blocks, 160), dtype=np.uint8)
    return out


def q6k_blocks(n_blocks: int, rng: np.random.Generator) -> np.ndarray:
    """Random Q6_K super-blocks (210 bytes: ql[128], qh[64], 16 signed scales, d;
    crates/modgrad-device/src/kfd/gguf.rs:458-466): quants uniform, scales uniform in [-128, 127],
    d = half(|N(0,1)| * 0.001)."""
    out = np.empty((n_blocks, 210), dtype=np.uint8)
    out[:, 0:208] = rng.integers(0, 256, size=(n_blocks, 208), dtype=np.uint8)
    d = (np.abs(rng.standard_normal((n_blocks, 1), dtype=np.float32)) * np.float32(0.001)).astype(np.float16)
    out[:, 208:210] = d.view(np.uint8).reshape(n_blocks, 2)
    return out


def kquant_matrix(kind: int, out_dim: int, in_dim: int, seed) -> np.ndarray:
    """Row-major Q5_K (kind 5) or Q6_K (kind 6) weight as a flat uint8 array."""
    assert in_dim % BLOCK_ELEMS == 0
    rng = seed if isinstance(seed, np.random.Generator) else np.random.Generator(np.random.PCG64(seed))
    gen = {5: q5k_blocks, 6: q6k_blocks}[kind]
    return gen(out_dim * (in_dim // BLOCK_ELEMS), rng).reshape(-1)


def q4k_matrix(out_dim: int, in_dim: int, seed) -> np.ndarray:
    """Row-major Q4_K weight ``[out_dim][in_dim/256][144]`` as a flat uint8 array."""
    assert in_dim % BLOCK_ELEMS == 0
    rng = seed if isinstance(seed, np.random.Generator) else np.random.Generator(np.random.PCG64(seed))
    return q4k_blocks(out_dim * (in_dim // BLOCK_ELEMS), rng).reshape(-1)


def activations(n: int, seed, rows: int | None = None) -> np.ndarray:
    """f32 N(0,1) activation vector (or ``rows`` x n matrix)."""
    rng = seed if isinstance(seed, np.random.Generator) else np.random.Generator(np.random.PCG64(seed))
    shape = (n,) if rows is None else (rows, n)
    return rng.standard_normal(shape, dtype=np.float32)


# Projection shapes (out_dim, in_dim) of the layer configurations the benchmark names.
QWEN25_7B_LAYER = {
    "q_proj": (3584, 3584), "k_proj": (512, 3584), "v_proj": (512, 3584), "o_proj": (3584, 3584),
    "gate_proj": (18944, 3584), "up_proj": (18944, 3584), "down_proj": (3584, 18944),
}
LLAMA_70B_LAYER = {
    "q_proj": (8192, 8192), "k_proj": (1024, 8192), "v_proj": (1024, 8192), "o_proj": (8192, 8192),
    "gate_proj": (28672, 8192), "up_proj": (28672, 8192), "down_proj": (8192, 28672),
}


def gemv_bytes(out_dim: int, in_dim: int) -> int:
    """Algorithmic bytes of one batch-1 Q4_K matvec: weights + x + y."""
    return out_dim * (in_dim // BLOCK_ELEMS) * BLOCK_BYTES + 4 * in_dim + 4 * out_dim

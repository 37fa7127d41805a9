"""Row sharding of the Q4_K path across the GPUs of one node (one process per GPU).

The reference has no multi-device code; the partition follows from the operation: output
rows are independent, so rank r of ``world`` holds a contiguous row range of every
projection — the unmodified row-major block array cut at row boundaries, nothing repacked —
and output slices are all-gathered (NCCL) where the next operation needs the whole vector.
The same arithmetic lives in ``mg_decoder_shard_ranges`` (C ABI).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np


def row_range(n: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous rows of rank ``rank``; remainders go to the first ranks."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


@dataclass(frozen=True)
class DecoderShard:
    rank: int
    world: int
    h0: int
    h1: int
    kv0: int
    kv1: int
    d_loc: int
    f_loc: int
    v_loc: int


def decoder_shard(cfg, rank: int, world: int) -> DecoderShard:
    """Head-parallel attention (q/k/v rows of a rank are whole heads), equal slices elsewhere."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    H, grp = cfg.n_heads, cfg.n_heads // cfg.n_kv_heads
    h0, h1 = rank * H // world, (rank + 1) * H // world
    if h1 <= h0:
        raise ValueError("more ranks than query heads")
    kv0, kv1 = h0 // grp, (h1 - 1) // grp + 1
    one_kv = (kv1 - kv0) == 1
    whole = h0 % grp == 0 and h1 % grp == 0
    if not (one_kv or whole):
        raise ValueError("a rank's query heads must be whole KV groups or share one KV head")
    if cfg.d_model % world or cfg.d_ff % world or (cfg.d_ff // world) % 64 or cfg.vocab % world:
        raise ValueError("hidden / FFN / vocabulary sizes must divide by the world size (FFN slice by 64)")
    return DecoderShard(rank, world, h0, h1, kv0, kv1, cfg.d_model // world, cfg.d_ff // world, cfg.vocab // world)


def q4k_rows(w: np.ndarray, out_dim: int, in_dim: int, lo: int, hi: int) -> np.ndarray:
    """Rows [lo, hi) of a row-major block-quantised matrix (Q4_K, Q5_K, Q6_K: whole rows of blocks), as bytes."""
    return np.ascontiguousarray(w.reshape(out_dim, w.size // out_dim)[lo:hi]).reshape(-1)


def slice_layer(cfg, sh: DecoderShard, lw: dict) -> dict:
    """This rank's slices of one layer's full tensors."""
    hd, D, F = cfg.head_dim, cfg.d_model, cfg.d_ff
    q_dim, kv_dim = cfg.n_heads * hd, cfg.n_kv_heads * hd
    r = sh.rank
    return {
        "wq": q4k_rows(lw["wq"], q_dim, D, sh.h0 * hd, sh.h1 * hd),
        "wk": q4k_rows(lw["wk"], kv_dim, D, sh.kv0 * hd, sh.kv1 * hd),
        "wv": q4k_rows(lw["wv"], kv_dim, D, sh.kv0 * hd, sh.kv1 * hd),
        "wo": q4k_rows(lw["wo"], D, q_dim, r * sh.d_loc, (r + 1) * sh.d_loc),
        "wgate": q4k_rows(lw["wgate"], F, D, r * sh.f_loc, (r + 1) * sh.f_loc),
        "wup": q4k_rows(lw["wup"], F, D, r * sh.f_loc, (r + 1) * sh.f_loc),
        "wdown": q4k_rows(lw["wdown"], D, F, r * sh.d_loc, (r + 1) * sh.d_loc),
        "attn_norm": lw["attn_norm"], "ffn_norm": lw["ffn_norm"],
    }


def slice_kv(cfg, sh: DecoderShard, kv: np.ndarray, n_pos: int) -> np.ndarray:
    hd = cfg.head_dim
    return np.ascontiguousarray(kv.reshape(n_pos, cfg.n_kv_heads * hd)[:, sh.kv0 * hd:sh.kv1 * hd]).reshape(-1)


def nccl_id_from_torch(rank: int) -> bytes:
    """Rank 0 makes an NCCL unique id through the C ABI; torch.distributed hands it round."""
    import torch.distributed as dist
    from . import _lib
    buf = (C.c_char * 128)()
    if rank == 0:
        code = _lib.load().mg_nccl_unique_id(buf)
        if code != 0:
            raise RuntimeError(f"mg_nccl_unique_id failed ({code}): is libnccl.so.2 loadable?")
    box = [bytes(buf) if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    return box[0]

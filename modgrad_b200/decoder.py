"""Python view of the resident Q4_K decoder engine (``mg_decoder_*`` in the C ABI).

Mirrors the reference's resident decode engine ``RocmGemma::{load, forward_token, generate}``
(crates/modgrad-gemma/src/rocm_gemma.rs:94, :312, :372); the arithmetic is that of the CPU
decoder ``kfd::llm::forward_token`` (crates/modgrad-device/src/kfd/llm.rs:1177-1298).
Weights are random-init synthetic tensors (there are no checkpoints to load): Q4_K
projections from ``synth.q4k_matrix``, half embedding / LM head N(0, 0.02), norm weights
1 + 0.05 N(0,1), an optional N(0,1) half KV prefill.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib, shard as shard_mod, synth
from .backend import Runtime

W_Q, W_K, W_V, W_O, W_GATE, W_UP, W_DOWN, W_ATTN_NORM, W_FFN_NORM = range(9)
W_EMBED, W_LM_HEAD, W_OUT_NORM = 100, 101, 102
Q4K_TENSORS = ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown")


class DecoderConfigC(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "d_ff",
                                       "vocab", "max_seq")] + [("rms_eps", C.c_float), ("rope_base", C.c_float)]


@dataclass
class DecoderConfig:
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    d_ff: int
    vocab: int
    max_seq: int
    rms_eps: float = 1e-6
    rope_base: float = 1e6

    @property
    def q_dim(self):
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self):
        return self.n_kv_heads * self.head_dim

    def shapes(self):
        """(out_dim, in_dim) of the seven Q4_K projections."""
        D, F = self.d_model, self.d_ff
        return {"wq": (self.q_dim, D), "wk": (self.kv_dim, D), "wv": (self.kv_dim, D), "wo": (D, self.q_dim),
                "wgate": (F, D), "wup": (F, D), "wdown": (D, F)}

    def q4k_bytes_per_layer(self):
        return sum(o * (i // 256) * 144 for o, i in self.shapes().values())

    def token_bytes(self, ctx: int) -> int:
        """Algorithmic bytes one decoded token reads: Q4_K weights, half LM head, half KV, one embedding row."""
        return (self.n_layers * self.q4k_bytes_per_layer() + self.vocab * self.d_model * 2
                + self.n_layers * 2 * ctx * self.kv_dim * 2 + self.d_model * 2)

    def c_struct(self):
        return DecoderConfigC(self.n_layers, self.d_model, self.n_heads, self.n_kv_heads, self.head_dim, self.d_ff,
                              self.vocab, self.max_seq, self.rms_eps, self.rope_base)


# The 7B-class architecture the benchmark names (Qwen2.5-7B dimensions).
QWEN25_7B = DecoderConfig(n_layers=28, d_model=3584, n_heads=28, n_kv_heads=4, head_dim=128, d_ff=18944,
                          vocab=152064, max_seq=2048 + 256 + 8)


def layer_weights(cfg: DecoderConfig, layer: int, seed: int):
    """Host tensors of one layer (deterministic per (seed, layer))."""
    rng = np.random.Generator(np.random.PCG64([seed, 1, layer]))
    out = {}
    for name, (o, i) in cfg.shapes().items():
        out[name] = synth.q4k_matrix(o, i, rng)
    out["attn_norm"] = (1.0 + 0.05 * rng.standard_normal(cfg.d_model, dtype=np.float32)).astype(np.float32)
    out["ffn_norm"] = (1.0 + 0.05 * rng.standard_normal(cfg.d_model, dtype=np.float32)).astype(np.float32)
    return out


def global_weights(cfg: DecoderConfig, seed: int):
    rng = np.random.Generator(np.random.PCG64([seed, 2]))
    n = cfg.vocab * cfg.d_model
    embed = (rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    lm_head = (rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    out_norm = (1.0 + 0.05 * rng.standard_normal(cfg.d_model, dtype=np.float32)).astype(np.float32)
    return {"embed": embed, "lm_head": lm_head, "out_norm": out_norm}


def kv_prefill(cfg: DecoderConfig, layer: int, n_pos: int, seed: int):
    rng = np.random.Generator(np.random.PCG64([seed, 3, layer]))
    k = rng.standard_normal(n_pos * cfg.kv_dim, dtype=np.float32).astype(np.float16)
    v = rng.standard_normal(n_pos * cfg.kv_dim, dtype=np.float32).astype(np.float16)
    return k, v


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class Q4KDecoder:
    """Device-resident decoder; one graph launch per token."""

    def __init__(self, cfg: DecoderConfig, rank: int = 0, world: int = 1, nccl_id: bytes | None = None,
                 types: tuple | None = None):
        """``types`` = (proj_types, embed_type, head_type) builds the typed engine: proj_types
        holds, per layer, the GGUF type ids (12 Q4_K, 13 Q5_K, 14 Q6_K) of q, k, v, o, gate, up, down;
        embed_type / head_type are 1 (F16) or one of the three."""
        self.cfg = cfg
        self.shard = shard_mod.decoder_shard(cfg, rank, world)
        self._lib = _lib.load()
        h = C.c_void_p()
        cs = cfg.c_struct()
        idbuf = C.create_string_buffer(nccl_id, 128) if nccl_id is not None else None
        if types is not None:
            proj, embed_type, head_type = types
            flat = np.ascontiguousarray(np.asarray(proj, dtype=np.int32).reshape(cfg.n_layers * 7))
            code = self._lib.mg_decoder_create_typed_sharded(C.byref(cs), _p(flat), int(embed_type), int(head_type), rank,
                                                             world, idbuf, C.byref(h))
        else:
            code = self._lib.mg_decoder_create_sharded(C.byref(cs), rank, world, idbuf, C.byref(h))
        if code != 0 or not h.value:
            raise Runtime(f"mg_decoder_create: {self._lib.mg_get_error_string(code).decode()}")
        self._h = h.value

    @classmethod
    def from_gguf(cls, path: str, max_seq: int, rank: int = 0, world: int = 1, nccl_id: bytes | None = None):
        """``RocmGemma::load``: configuration from the file's metadata, every tensor uploaded verbatim
        from the memory-mapped file (this rank's row ranges), behind the VRAM guard."""
        from . import gguf
        lib = _lib.load()
        with gguf.GgufFile.open(path) as g:
            cs = DecoderConfigC()
            if lib.mg_decoder_config_from_gguf(g.handle, max_seq, C.byref(cs)) != 0:
                raise Runtime(f"gguf config: {lib.mg_decoder_load_error().decode()}")
        cfg = DecoderConfig(cs.n_layers, cs.d_model, cs.n_heads, cs.n_kv_heads, cs.head_dim, cs.d_ff, cs.vocab,
                            cs.max_seq, cs.rms_eps, cs.rope_base)
        self = cls.__new__(cls)
        self.cfg = cfg
        self.shard = shard_mod.decoder_shard(cfg, rank, world)
        self._lib = lib
        h = C.c_void_p()
        idbuf = C.create_string_buffer(nccl_id, 128) if nccl_id is not None else None
        code = lib.mg_decoder_load_gguf(str(path).encode(), max_seq, rank, world, idbuf, C.byref(h))
        if code != 0 or not h.value:
            from .backend import OutOfMemory
            msg = lib.mg_decoder_load_error().decode()
            raise (OutOfMemory if code == 2 else Runtime)(f"load_gguf: {msg}")
        self._h = h.value
        self.set_position(0)
        return self

    def weight_arena(self) -> tuple[int, int]:
        """(base device pointer, bytes) of the single allocation that holds every weight tensor."""
        n = C.c_size_t()
        return int(self._lib.mg_decoder_weight_arena(self._h, C.byref(n)) or 0), n.value

    def weight_type(self, layer: int, which: int) -> int:
        """GGUF type id of one weight tensor (0 for the f32 norms)."""
        return int(self._lib.mg_decoder_weight_type(self._h, layer, which))

    def weight_ptr(self, layer: int, which: int) -> int:
        return int(self._lib.mg_decoder_weight_ptr(self._h, layer, which) or 0)

    def close(self):
        if getattr(self, "_h", None):
            self._lib.mg_decoder_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, code: int, what: str):
        if code != 0:
            msg = self._lib.mg_decoder_last_error(self._h).decode() or self._lib.mg_get_error_string(code).decode()
            raise Runtime(f"{what}: {msg}")

    def upload(self, layer: int, which: int, a: np.ndarray):
        a = np.ascontiguousarray(a)
        self._check(self._lib.mg_decoder_upload(self._h, layer, which, _p(a), a.nbytes), "upload")

    def load_random(self, seed: int, prefill: int = 0, on_layer=None):
        """RocmGemma::load for random-init weights: generate on the host, upload verbatim.
        With world > 1 every rank generates the same full tensors and uploads its row slices."""
        cfg, sh = self.cfg, self.shard
        g = global_weights(cfg, seed)
        self.upload(0, W_EMBED, g["embed"])
        self.upload(0, W_LM_HEAD, g["lm_head"].reshape(cfg.vocab, cfg.d_model)[sh.rank * sh.v_loc:(sh.rank + 1) * sh.v_loc])
        self.upload(0, W_OUT_NORM, g["out_norm"])
        for l in range(cfg.n_layers):
            lw = layer_weights(cfg, l, seed)
            mine = shard_mod.slice_layer(cfg, sh, lw) if sh.world > 1 else lw
            for idx, name in enumerate(Q4K_TENSORS):
                self.upload(l, idx, mine[name])
            self.upload(l, W_ATTN_NORM, lw["attn_norm"])
            self.upload(l, W_FFN_NORM, lw["ffn_norm"])
            if prefill:
                k, v = kv_prefill(cfg, l, prefill, seed)
                if sh.world > 1:
                    k, v = shard_mod.slice_kv(cfg, sh, k, prefill), shard_mod.slice_kv(cfg, sh, v, prefill)
                self.set_kv(l, k, v, prefill)
            if on_layer:
                on_layer(l, lw)
        if not prefill:
            self.set_position(0)
        return g

    def load_random_shard(self, seed: int, prefill: int = 0):
        """Benchmark loader: this rank's slices generated directly (seeded per rank), so that no
        rank has to build the whole model on the host.  Same shapes and value distributions."""
        cfg, sh = self.cfg, self.shard
        hd, D, F = cfg.head_dim, cfg.d_model, cfg.d_ff
        rng = np.random.Generator(np.random.PCG64([seed, 9, sh.rank]))
        n = cfg.vocab * D
        self.upload(0, W_EMBED, (rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)).astype(np.float16))
        self.upload(0, W_LM_HEAD, (rng.standard_normal(sh.v_loc * D, dtype=np.float32) * np.float32(0.02)).astype(np.float16))
        norm = (1.0 + 0.05 * np.random.Generator(np.random.PCG64([seed, 8])).standard_normal(D, dtype=np.float32)).astype(np.float32)
        self.upload(0, W_OUT_NORM, norm)
        q_loc, kv_loc = (sh.h1 - sh.h0) * hd, (sh.kv1 - sh.kv0) * hd
        dims = {"wq": (q_loc, D), "wk": (kv_loc, D), "wv": (kv_loc, D), "wo": (sh.d_loc, cfg.q_dim),
                "wgate": (sh.f_loc, D), "wup": (sh.f_loc, D), "wdown": (sh.d_loc, F)}
        for l in range(cfg.n_layers):
            for idx, name in enumerate(Q4K_TENSORS):
                o, i = dims[name]
                self.upload(l, idx, synth.q4k_matrix(o, i, rng))
            self.upload(l, W_ATTN_NORM, norm)
            self.upload(l, W_FFN_NORM, norm)
            if prefill:
                k = rng.standard_normal(prefill * kv_loc, dtype=np.float32).astype(np.float16)
                v = rng.standard_normal(prefill * kv_loc, dtype=np.float32).astype(np.float16)
                self.set_kv(l, k, v, prefill)
        if not prefill:
            self.set_position(0)

    def set_kv(self, layer: int, k: np.ndarray, v: np.ndarray, n_pos: int):
        k, v = np.ascontiguousarray(k), np.ascontiguousarray(v)
        self._check(self._lib.mg_decoder_set_kv(self._h, layer, _p(k), _p(v), n_pos), "set_kv")

    def set_position(self, pos: int):
        self._check(self._lib.mg_decoder_set_position(self._h, pos), "set_position")

    def forward_token(self, token: int, want_logits: bool = True):
        logits = np.empty(self.shard.v_loc, dtype=np.float32) if want_logits else None  # this rank's slice
        nxt = C.c_int(0)
        self._check(self._lib.mg_decoder_forward_token(self._h, int(token), _p(logits) if want_logits else None,
                                                       C.byref(nxt)), "forward_token")
        return logits, nxt.value

    def generate(self, first_token: int, n_tokens: int):
        """Greedy decode; returns (tokens, device milliseconds)."""
        out = np.empty(n_tokens, dtype=np.int32)
        ms = C.c_float(0)
        self._check(self._lib.mg_decoder_generate(self._h, int(first_token), n_tokens, _p(out), C.byref(ms)), "generate")
        return out, float(ms.value)

    def set_exchange_spin_limit(self, polls: int):
        """Polls a bounded wait of the peer exchanges makes before the token fails (before the first token)."""
        self._check(self._lib.mg_decoder_set_exchange_spin_limit(self._h, int(polls)), "set_exchange_spin_limit")

    def kernels_per_token(self) -> int:
        return int(self._lib.mg_decoder_kernels_per_token(self._h))

    def gather_mode(self) -> str:
        """How a sharded engine all-gathers its slices: "nccl", "peer" (one peer-store gather
        kernel per collective), "fused" (inside the producing kernels, flag handshake at their end) or
        "stamped" (inside the producing kernels, every word carrying its epoch); "none" on one GPU."""
        return {-1: "none", 0: "nccl", 1: "peer", 2: "fused", 3: "stamped"}[int(self._lib.mg_decoder_gather_mode(self._h))]

"""ctypes loader for the C oracle (oracle/q4k_oracle.c, oracle/decoder_oracle.c).

Test infrastructure only: nothing under modgrad_b200/ may import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_build" / "libq4k_oracle.so"

MODE_SCALAR, MODE_SELECT, MODE_F64 = 0, 1, 2


def build(force: bool = False) -> Path:
    """Compile the oracle with the committed Makefile (gcc, -ffp-contract=off)."""
    srcs = [_HERE / "q4k_oracle.c", _HERE / "decoder_oracle.c", _HERE / "kquant_oracle.c", _HERE / "Makefile"]
    stale = (not _SO.exists()) or any(s.stat().st_mtime > _SO.stat().st_mtime for s in srcs)
    if force or stale:
        subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


class DecoderCfg(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim",
                                       "d_ff", "vocab", "max_seq")] + \
               [("rms_eps", C.c_float), ("rope_base", C.c_float)]


class DecoderLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown",
                                          "attn_norm", "ffn_norm", "k_cache", "v_cache")]


class TypedLayer(C.Structure):
    """orc_typed_layer: seven weight pointers (wq, wk, wv, wo, wgate, wup, wdown), their GGML type ids,
    the two norm vectors and the half KV caches."""
    _fields_ = [("w", C.c_void_p * 7), ("type", C.c_int * 7), ("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p),
                ("k_cache", C.c_void_p), ("v_cache", C.c_void_p)]


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class OracleLib:
    def __init__(self, path: Path):
        self.c = C.CDLL(str(path))
        c = self.c
        c.orc_f16_to_f32.restype = C.c_float
        c.orc_f16_to_f32.argtypes = [C.c_uint16]
        c.orc_f32_to_f16_rne.restype = C.c_uint16
        c.orc_f32_to_f16_rne.argtypes = [C.c_float]
        c.orc_get_scale_min_k4.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        c.orc_pack_scales_mins.argtypes = [C.c_void_p] * 3
        c.orc_dequantize_row_q4_k.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        for f in (c.orc_dot_q4k_row_scalar, c.orc_dot_q4k_row):
            f.restype = C.c_float
            f.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        c.orc_dot_q4k_row_f64.restype = C.c_double
        c.orc_dot_q4k_row_f64.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        c.orc_matvec_q4k.restype = C.c_int
        c.orc_matvec_q4k.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]
        c.orc_matvec_q4k_f64.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        c.orc_quantize_q8_1.argtypes = [C.c_void_p] * 4 + [C.c_int]
        c.orc_matvec_q4k_q8_1.argtypes = [C.c_void_p] * 5 + [C.c_int, C.c_int]
        c.orc_dequantize_row_q5_k.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        c.orc_dequantize_row_q6_k.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        c.orc_matvec_kquant_f64.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        c.orc_matvec_q6k_q8_1.argtypes = [C.c_void_p] * 4 + [C.c_int, C.c_int]
        c.orc_rms_norm.argtypes = [C.c_void_p] * 3 + [C.c_int, C.c_float]
        c.orc_apply_rope.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float]
        c.orc_attention_f16kv.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4
        c.orc_swiglu_inplace.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        c.orc_matvec_f16.argtypes = [C.c_void_p] * 3 + [C.c_int, C.c_int]
        c.orc_argmax.restype = C.c_uint32
        c.orc_argmax.argtypes = [C.c_void_p, C.c_int]
        c.orc_forward_token.argtypes = [C.c_void_p] * 5 + [C.c_int, C.c_uint32, C.c_void_p, C.c_int]
        c.orc_forward_token_typed.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                              C.c_int, C.c_uint32, C.c_void_p]
        c.orc_forward_token_typed.restype = None
        c.orc_forward_token_f32kv.argtypes = [C.c_void_p] * 7 + [C.c_int, C.c_uint32, C.c_void_p, C.c_int]

    # ---- format -----------------------------------------------------------------------
    def f16_to_f32(self, h: int) -> float:
        return float(self.c.orc_f16_to_f32(h))

    def get_scale_min_k4(self, j: int, scales: np.ndarray):
        sc, m = C.c_uint8(), C.c_uint8()
        s = np.ascontiguousarray(scales, dtype=np.uint8)
        self.c.orc_get_scale_min_k4(j, _p(s), C.byref(sc), C.byref(m))
        return sc.value, m.value

    def dequantize(self, blocks: np.ndarray) -> np.ndarray:
        b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        n = b.size // 144
        out = np.empty(n * 256, dtype=np.float32)
        self.c.orc_dequantize_row_q4_k(_p(b), _p(out), n)
        return out

    def dequantize_kquant(self, kind: int, blocks: np.ndarray) -> np.ndarray:
        """kind 5: Q5_K (176-byte blocks), 6: Q6_K (210-byte blocks)."""
        bb = {5: 176, 6: 210}[kind]
        b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        n = b.size // bb
        out = np.empty(n * 256, dtype=np.float32)
        (self.c.orc_dequantize_row_q5_k if kind == 5 else self.c.orc_dequantize_row_q6_k)(_p(b), _p(out), n)
        return out

    def matvec_kquant_f64(self, kind: int, w: np.ndarray, x: np.ndarray, out_dim: int, bpr: int) -> np.ndarray:
        bb = {5: 176, 6: 210}[kind]
        w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1)
        x = np.ascontiguousarray(x, dtype=np.float32)
        assert w.size == out_dim * bpr * bb and x.size >= bpr * 256
        y = np.empty(out_dim, dtype=np.float64)
        self.c.orc_matvec_kquant_f64(kind, _p(w), _p(x), _p(y), out_dim, bpr)
        return y

    def matvec_q6k_q8_1(self, w, xq, xd, out_dim, bpr):
        w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1)
        y = np.empty(out_dim, dtype=np.float32)
        self.c.orc_matvec_q6k_q8_1(_p(w), _p(xq), _p(xd), _p(y), out_dim, bpr)
        return y

    # ---- matvec -----------------------------------------------------------------------
    def matvec(self, w: np.ndarray, x: np.ndarray, out_dim: int, bpr: int, mode: int = MODE_F64,
               threads: int = 0) -> np.ndarray:
        w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1)
        x = np.ascontiguousarray(x, dtype=np.float32)
        assert w.size == out_dim * bpr * 144 and x.size >= bpr * 256
        y = np.empty(out_dim, dtype=np.float32)
        self.c.orc_matvec_q4k(_p(w), _p(x), _p(y), out_dim, bpr, mode, threads)
        return y

    def matvec_f64(self, w: np.ndarray, x: np.ndarray, out_dim: int, bpr: int) -> np.ndarray:
        w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1)
        x = np.ascontiguousarray(x, dtype=np.float32)
        assert w.size == out_dim * bpr * 144 and x.size >= bpr * 256
        y = np.empty(out_dim, dtype=np.float64)
        self.c.orc_matvec_q4k_f64(_p(w), _p(x), _p(y), out_dim, bpr, 0)
        return y

    def max_threads(self) -> int:
        return int(self.c.orc_max_threads())

    def has_avx512(self) -> bool:
        return bool(self.c.orc_has_avx512())

    # ---- int8-activation side path ------------------------------------------------------
    def quantize_q8_1(self, x: np.ndarray):
        x = np.ascontiguousarray(x, dtype=np.float32)
        n = x.size
        xq = np.empty(n, dtype=np.int8)
        xd = np.empty(n // 32, dtype=np.float32)
        xs = np.empty(n // 32, dtype=np.float32)
        self.c.orc_quantize_q8_1(_p(x), _p(xq), _p(xd), _p(xs), n)
        return xq, xd, xs

    def matvec_q8_1(self, w, xq, xd, xs, out_dim, bpr):
        w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1)
        y = np.empty(out_dim, dtype=np.float32)
        self.c.orc_matvec_q4k_q8_1(_p(w), _p(xq), _p(xd), _p(xs), _p(y), out_dim, bpr)
        return y

    # ---- decoder glue -------------------------------------------------------------------
    def rms_norm(self, x, w, eps):
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        y = np.empty_like(x)
        self.c.orc_rms_norm(_p(x), _p(w), _p(y), x.size, eps)
        return y

    def apply_rope(self, data, pos, n_heads, head_dim, base):
        d = np.array(data, dtype=np.float32, copy=True)
        self.c.orc_apply_rope(_p(d), pos, n_heads, head_dim, base)
        return d

    def attention_f16kv(self, q, k_buf, v_buf, seq_len, n_heads, n_kv_heads, head_dim):
        q = np.ascontiguousarray(q, dtype=np.float32)
        k = np.ascontiguousarray(k_buf).view(np.uint16)
        v = np.ascontiguousarray(v_buf).view(np.uint16)
        out = np.empty(n_heads * head_dim, dtype=np.float32)
        self.c.orc_attention_f16kv(_p(q), _p(k), _p(v), _p(out), seq_len, n_heads, n_kv_heads, head_dim)
        return out

    def swiglu(self, gate, up):
        g = np.array(gate, dtype=np.float32, copy=True)
        u = np.ascontiguousarray(up, dtype=np.float32)
        self.c.orc_swiglu_inplace(_p(g), _p(u), g.size)
        return g

    def matvec_f16(self, w, x, out_dim, in_dim):
        w = np.ascontiguousarray(w).view(np.uint16)
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(out_dim, dtype=np.float32)
        self.c.orc_matvec_f16(_p(w), _p(x), _p(y), out_dim, in_dim)
        return y

    def argmax(self, v) -> int:
        v = np.ascontiguousarray(v, dtype=np.float32)
        return int(self.c.orc_argmax(_p(v), v.size))

    def forward_token(self, cfg: DecoderCfg, layers, embed, lm_head, out_norm, pos, token,
                      mode: int = MODE_F64) -> np.ndarray:
        arr = (DecoderLayer * len(layers))(*layers)
        logits = np.empty(cfg.vocab, dtype=np.float32)
        self.c.orc_forward_token(C.byref(cfg), arr, _p(embed), _p(lm_head), _p(out_norm), pos, token,
                                 _p(logits), mode)
        return logits

    def forward_token_typed(self, cfg: DecoderCfg, layers, embed, embed_type, lm_head, head_type, out_norm, pos,
                            token) -> np.ndarray:
        """forward_token over tensors of mixed GGML types (layers: TypedLayer records; type ids 1 F16, 12 Q4_K,
        13 Q5_K, 14 Q6_K), f64-accumulated matvecs, half KV caches appended in place."""
        arr = (TypedLayer * len(layers))(*layers)
        logits = np.empty(cfg.vocab, dtype=np.float32)
        self.c.orc_forward_token_typed(C.byref(cfg), arr, _p(embed), int(embed_type), _p(lm_head), int(head_type),
                                       _p(out_norm), pos, token, _p(logits))
        return logits

    def forward_token_f32kv(self, cfg: DecoderCfg, layers, k32, v32, embed, lm_head, out_norm, pos, token,
                            mode: int = MODE_F64) -> np.ndarray:
        """The reference's own arrangement: f32 KV caches (k32[l], v32[l]: [max_seq * kv_dim] f32 arrays,
        appended unrounded, crates/modgrad-device/src/kfd/llm.rs:305-310, :1232-1234)."""
        arr = (DecoderLayer * len(layers))(*layers)
        kp = (C.c_void_p * len(k32))(*[a.ctypes.data for a in k32])
        vp_ = (C.c_void_p * len(v32))(*[a.ctypes.data for a in v32])
        logits = np.empty(cfg.vocab, dtype=np.float32)
        self.c.orc_forward_token_f32kv(C.byref(cfg), arr, kp, vp_, _p(embed), _p(lm_head), _p(out_norm), pos, token,
                                       _p(logits), mode)
        return logits


_LIB = None


def lib() -> OracleLib:
    global _LIB
    if _LIB is None:
        if not _SO.exists() or os.environ.get("Q4K_ORACLE_REBUILD"):
            build()
        _LIB = OracleLib(_SO)
    return _LIB

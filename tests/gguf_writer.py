"""Minimal GGUF v3 (or v2) writer for the tests: header, metadata key/values, tensor infos, data
section aligned to 32 bytes.  Follows the layout the reference parser reads
(crates/modgrad-device/src/kfd/gguf.rs:153-208, :665-694).  Test infrastructure only."""
from __future__ import annotations

import struct

import numpy as np

T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_FMT = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<B",
        T_U64: "<Q", T_I64: "<q", T_F64: "<d"}
GGML_F32, GGML_F16, GGML_Q4_K, GGML_Q5_K, GGML_Q6_K = 0, 1, 12, 13, 14


def _string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _value(vtype: int, v) -> bytes:
    if vtype == T_STR:
        return _string(v)
    if vtype == T_ARR:
        atype, items = v
        return struct.pack("<IQ", atype, len(items)) + b"".join(_value(atype, x) for x in items)
    return struct.pack(_FMT[vtype], v)


def write_gguf(meta: list, tensors: list, version: int = 3, align: int = 32) -> bytes:
    """meta: [(key, vtype, value)], tensors: [(name, dims (dims[0] fastest), ggml dtype, bytes-like)]."""
    out = bytearray(b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(meta)))
    for key, vtype, v in meta:
        out += _string(key) + struct.pack("<I", vtype) + _value(vtype, v)
    blobs, off = [], 0
    for name, dims, dtype, data in tensors:
        data = bytes(memoryview(np.ascontiguousarray(data)).cast("B"))
        out += _string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", dtype, off)
        blobs.append((off, data))
        off = (off + len(data) + align - 1) // align * align
    out += b"\0" * ((-len(out)) % 32)
    base = len(out)
    for o, data in blobs:
        out += b"\0" * (base + o - len(out)) + data
    return bytes(out)


def decoder_gguf(cfg, layers: list, g: dict, arch: str = "qwen2", tied: bool = False) -> bytes:
    """A checkpoint of the decoder architecture the engine runs, from host tensors:
    layers[l] = dict(wq, wk, wv, wo, wgate, wup, wdown, attn_norm, ffn_norm), g = dict(embed, lm_head, out_norm).
    A layer's optional "types" maps a projection key to its GGML type (default Q4_K); g's optional
    "embed_type" / "head_type" give the types of the embedding and the LM head (default F16)."""
    meta = [("general.architecture", T_STR, arch), (f"{arch}.block_count", T_U32, cfg.n_layers),
            (f"{arch}.embedding_length", T_U32, cfg.d_model), (f"{arch}.feed_forward_length", T_U32, cfg.d_ff),
            (f"{arch}.attention.head_count", T_U32, cfg.n_heads), (f"{arch}.attention.head_count_kv", T_U32, cfg.n_kv_heads),
            (f"{arch}.attention.key_length", T_U32, cfg.head_dim),
            (f"{arch}.attention.layer_norm_rms_epsilon", T_F32, cfg.rms_eps), (f"{arch}.rope.freq_base", T_F32, cfg.rope_base),
            ("tokenizer.ggml.tokens", T_ARR, (T_STR, ["<a>", "<b>", "c"])), ("general.alignment", T_U32, 32)]
    D, F = cfg.d_model, cfg.d_ff
    ts = [("token_embd.weight", (D, cfg.vocab), g.get("embed_type", GGML_F16), g["embed"])]
    names = {"wq": ("attn_q", D, cfg.q_dim), "wk": ("attn_k", D, cfg.kv_dim), "wv": ("attn_v", D, cfg.kv_dim),
             "wo": ("attn_output", cfg.q_dim, D), "wgate": ("ffn_gate", D, F), "wup": ("ffn_up", D, F),
             "wdown": ("ffn_down", F, D)}
    for l, lw in enumerate(layers):
        for k, (n, i, o) in names.items():
            ts.append((f"blk.{l}.{n}.weight", (i, o), lw.get("types", {}).get(k, GGML_Q4_K), lw[k]))
        ts.append((f"blk.{l}.attn_norm.weight", (D,), GGML_F32, lw["attn_norm"]))
        ts.append((f"blk.{l}.ffn_norm.weight", (D,), GGML_F32, lw["ffn_norm"]))
    ts.append(("output_norm.weight", (D,), GGML_F32, g["out_norm"]))
    if not tied:
        ts.append(("output.weight", (D, cfg.vocab), g.get("head_type", GGML_F16), g["lm_head"]))
    return write_gguf(meta, ts)

"""The oracle's forward pass over tensors of mixed types (orc_forward_token_typed: the type dispatch of the
reference's matvec, crates/modgrad-device/src/kfd/llm.rs:498-533, and its quantised embedding lookup, :898-918)
against the same pass composed step by step from the oracle's pieces, and against orc_forward_token where all
types are the defaults."""
import ctypes as C

import numpy as np

from modgrad_b200 import decoder as dec
from oracle.loader import MODE_F64, DecoderCfg, DecoderLayer, TypedLayer
from test_gpu_decoder_typed import F16, MIX, Q4, Q5, Q6, SMALL, mixed_model, oracle_forward


def typed_layers(cfg, layers, caches):
    p = lambda a: a.ctypes.data_as(C.c_void_p).value
    out = []
    for lw, (kc, vc) in zip(layers, caches):
        t = TypedLayer()
        for i, name in enumerate(dec.Q4K_TENSORS):
            t.w[i] = p(lw[name])
            t.type[i] = lw["types"][name]
        t.attn_norm, t.ffn_norm, t.k_cache, t.v_cache = p(lw["attn_norm"]), p(lw["ffn_norm"]), p(kc), p(vc)
        out.append(t)
    return out


def fresh_caches(cfg):
    return [(np.zeros(cfg.max_seq * cfg.kv_dim, dtype=np.float16), np.zeros(cfg.max_seq * cfg.kv_dim, dtype=np.float16))
            for _ in range(cfg.n_layers)]


def c_cfg(cfg):
    return DecoderCfg(cfg.n_layers, cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.d_ff, cfg.vocab,
                      cfg.max_seq, cfg.rms_eps, cfg.rope_base)


def test_typed_forward_equals_the_step_by_step_composition(orc):
    cfg = SMALL
    for embed_type, head_type in ((Q6, Q6), (Q4, F16), (F16, Q5)):
        layers, g = mixed_model(cfg, 61, MIX, embed_type, head_type)
        ca, cb = fresh_caches(cfg), fresh_caches(cfg)
        tl = typed_layers(cfg, layers, ca)
        for pos, tok in enumerate([3, 600, 77]):
            got = orc.forward_token_typed(c_cfg(cfg), tl, g["embed"], embed_type, g["lm_head"], head_type, g["out_norm"], pos, tok)
            want = oracle_forward(orc, cfg, layers, g, cb, pos, tok)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (embed_type, head_type, pos)
        for (ka, va), (kb, vb) in zip(ca, cb):
            assert np.array_equal(ka.view(np.uint16), kb.view(np.uint16)) and np.array_equal(va.view(np.uint16), vb.view(np.uint16))


def test_typed_forward_with_default_types_is_forward_token(orc):
    cfg, seed = SMALL, 62
    layers = [dict(dec.layer_weights(cfg, l, seed), types={n: Q4 for n in dec.Q4K_TENSORS}) for l in range(cfg.n_layers)]
    g = dec.global_weights(cfg, seed)
    ca, cb = fresh_caches(cfg), fresh_caches(cfg)
    tl = typed_layers(cfg, layers, ca)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    plain = [DecoderLayer(*[p(lw[n]) for n in dec.Q4K_TENSORS], p(lw["attn_norm"]), p(lw["ffn_norm"]), p(kc), p(vc))
             for lw, (kc, vc) in zip(layers, cb)]
    for pos, tok in enumerate([9, 311]):
        a = orc.forward_token_typed(c_cfg(cfg), tl, g["embed"], F16, g["lm_head"], F16, g["out_norm"], pos, tok)
        b = orc.forward_token(c_cfg(cfg), plain, g["embed"], g["lm_head"], g["out_norm"], pos, tok, MODE_F64)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), pos

"""The typed engine: projections, token embedding and LM head in the mix of K-quants a real checkpoint
carries (Q4_K with Q6_K attn_v / ffn_down / embedding / head and some Q5_K; the per-tensor dispatch of
crates/modgrad-gemma/src/rocm_gemma.rs:291-309), against a forward pass composed from the CPU oracle's
pieces in the order of kfd::llm::forward_token (crates/modgrad-device/src/kfd/llm.rs:1177-1298)."""
import ctypes as C

import numpy as np
import pytest

import gguf_writer as gw
from conftest import rel_rms_err
from modgrad_b200 import decoder as dec
from modgrad_b200 import synth
from modgrad_b200.backend import DeviceBuffer, Runtime, kern

pytestmark = pytest.mark.gpu

DECODER_TOL = 1e-3   # logits after whole layers: reordered f32 sums compound through the depth
Q4, Q5, Q6, F16 = 12, 13, 14, 1
KIND = {Q5: 5, Q6: 6}
SMALL = dec.DecoderConfig(n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, d_ff=1024, vocab=640,
                          max_seq=40, rms_eps=1e-6, rope_base=1e6)
# per layer: types of q, k, v, o, gate, up, down
MIX = [[Q4, Q5, Q6, Q4, Q4, Q4, Q6],
       [Q4, Q4, Q4, Q5, Q6, Q4, Q4]]


def typed_matrix(t, rows, cols, rng):
    if t == Q4:
        return synth.q4k_matrix(rows, cols, rng)
    if t == F16:
        return (rng.standard_normal(rows * cols, dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    return synth.kquant_matrix(KIND[t], rows, cols, rng)


def mixed_model(cfg, seed, mix, embed_type, head_type):
    layers = []
    for l in range(cfg.n_layers):
        rng = np.random.Generator(np.random.PCG64([seed, 1, l]))
        lw = {"types": {}}
        for i, (name, (o, n_in)) in enumerate(cfg.shapes().items()):
            lw[name] = typed_matrix(mix[l][i], o, n_in, rng)
            lw["types"][name] = mix[l][i]
        lw["attn_norm"] = (1.0 + 0.05 * rng.standard_normal(cfg.d_model, dtype=np.float32)).astype(np.float32)
        lw["ffn_norm"] = (1.0 + 0.05 * rng.standard_normal(cfg.d_model, dtype=np.float32)).astype(np.float32)
        layers.append(lw)
    rng = np.random.Generator(np.random.PCG64([seed, 2]))
    g = {"embed": typed_matrix(embed_type, cfg.vocab, cfg.d_model, rng), "embed_type": embed_type,
         "lm_head": typed_matrix(head_type, cfg.vocab, cfg.d_model, rng), "head_type": head_type,
         "out_norm": (1.0 + 0.05 * rng.standard_normal(cfg.d_model, dtype=np.float32)).astype(np.float32)}
    return layers, g


def oracle_matvec(orc, t, w, x, rows, cols):
    if t == Q4:
        return orc.matvec_f64(w, x, rows, cols // 256).astype(np.float32)
    if t == F16:
        return orc.matvec_f16(w, x, rows, cols)
    return orc.matvec_kquant_f64(KIND[t], w, x, rows, cols // 256).astype(np.float32)


def oracle_row(orc, t, table, row, cols):
    if t == F16:
        return table.reshape(-1, cols)[row].astype(np.float32)
    bb = {Q4: 144, Q5: 176, Q6: 210}[t]
    blocks = table.reshape(-1, cols // 256 * bb)[row]
    return orc.dequantize(blocks) if t == Q4 else orc.dequantize_kquant(KIND[t], blocks)


def oracle_forward(orc, cfg, layers, g, caches, pos, token):
    """One token; caches[l] = (k, v) half arrays [max_seq * kv_dim], appended in place."""
    D, hd, F = cfg.d_model, cfg.head_dim, cfg.d_ff
    hidden = oracle_row(orc, g["embed_type"], g["embed"], token, D).copy()
    for l, lw in enumerate(layers):
        t = lw["types"]
        cur = orc.rms_norm(hidden, lw["attn_norm"], cfg.rms_eps)
        q = oracle_matvec(orc, t["wq"], lw["wq"], cur, cfg.q_dim, D)
        k = oracle_matvec(orc, t["wk"], lw["wk"], cur, cfg.kv_dim, D)
        v = oracle_matvec(orc, t["wv"], lw["wv"], cur, cfg.kv_dim, D)
        q = orc.apply_rope(q, pos, cfg.n_heads, hd, cfg.rope_base)
        k = orc.apply_rope(k, pos, cfg.n_kv_heads, hd, cfg.rope_base)
        kc, vc = caches[l]
        kc[pos * cfg.kv_dim:(pos + 1) * cfg.kv_dim] = k.astype(np.float16)
        vc[pos * cfg.kv_dim:(pos + 1) * cfg.kv_dim] = v.astype(np.float16)
        att = orc.attention_f16kv(q, kc, vc, pos + 1, cfg.n_heads, cfg.n_kv_heads, hd)
        hidden = hidden + oracle_matvec(orc, t["wo"], lw["wo"], att, D, cfg.q_dim)
        cur = orc.rms_norm(hidden, lw["ffn_norm"], cfg.rms_eps)
        gate = oracle_matvec(orc, t["wgate"], lw["wgate"], cur, F, D)
        upv = oracle_matvec(orc, t["wup"], lw["wup"], cur, F, D)
        act = orc.swiglu(gate, upv)
        hidden = hidden + oracle_matvec(orc, t["wdown"], lw["wdown"], act, D, F)
    cur = orc.rms_norm(hidden, g["out_norm"], cfg.rms_eps)
    return oracle_matvec(orc, g["head_type"], g["lm_head"], cur, cfg.vocab, D)


def upload_model(d, cfg, layers, g):
    d.upload(0, dec.W_EMBED, g["embed"])
    d.upload(0, dec.W_LM_HEAD, g["lm_head"])
    d.upload(0, dec.W_OUT_NORM, g["out_norm"])
    for l, lw in enumerate(layers):
        for idx, name in enumerate(dec.Q4K_TENSORS):
            d.upload(l, idx, lw[name])
        d.upload(l, dec.W_ATTN_NORM, lw["attn_norm"])
        d.upload(l, dec.W_FFN_NORM, lw["ffn_norm"])
    d.set_position(0)


@pytest.mark.parametrize("t", [Q4, Q5, Q6])
def test_quantised_embedding_row_is_the_bulk_dequantisation(orc, cuda, t):
    rng = np.random.Generator(np.random.PCG64(31 + t))
    vocab, D = 300, 768
    table = typed_matrix(t, vocab, D, rng)
    td = DeviceBuffer(table.nbytes)
    td.copy_from_host_bytes(table)
    out, tok = DeviceBuffer(D * 4), DeviceBuffer(4)
    host = np.empty(D, dtype=np.float32)
    from modgrad_b200 import _lib
    for row, from_device in ((0, False), (299, False), (123, True), (5000, False)):   # the last one clamps to vocab - 1
        if from_device:
            tok.copy_from_host_bytes(np.array([row], dtype=np.int32))
        assert cuda.mg_embed_kquant_on_stream(td.ptr, t, 0 if from_device else row, tok.ptr if from_device else None,
                                              out.ptr, D, vocab, None) == 0
        kern.sync()
        assert _lib.load().mg_memcpy_d2h(host.ctypes.data_as(C.c_void_p), out.ptr, host.nbytes) == 0
        want = oracle_row(orc, t, table, min(row, vocab - 1), D)
        assert np.array_equal(host.view(np.uint32), want.view(np.uint32)), (t, row)
    assert cuda.mg_embed_kquant_on_stream(td.ptr, 2, 0, None, out.ptr, D, vocab, None) != 0      # Q4_0: no kernel
    assert cuda.mg_embed_kquant_on_stream(td.ptr, t, 0, None, out.ptr, D + 32, vocab, None) != 0  # ragged row


@pytest.mark.parametrize("embed_type,head_type", [(Q6, Q6), (Q4, F16), (F16, Q5)])
def test_typed_engine_logits_match_oracle_teacher_forced(orc, embed_type, head_type):
    cfg, seed = SMALL, 41
    layers, g = mixed_model(cfg, seed, MIX, embed_type, head_type)
    d = dec.Q4KDecoder(cfg, types=(MIX, embed_type, head_type))
    assert d.weight_type(0, dec.W_V) == Q6 and d.weight_type(1, dec.W_O) == Q5 and d.weight_type(1, dec.W_Q) == Q4
    assert d.weight_type(0, dec.W_EMBED) == embed_type and d.weight_type(0, dec.W_LM_HEAD) == head_type
    assert d.weight_type(0, dec.W_ATTN_NORM) == 0
    upload_model(d, cfg, layers, g)
    caches = [(np.zeros(cfg.max_seq * cfg.kv_dim, dtype=np.float16), np.zeros(cfg.max_seq * cfg.kv_dim, dtype=np.float16))
              for _ in range(cfg.n_layers)]
    for pos, tok in enumerate([3, 600, 77, 5, 311]):
        want = oracle_forward(orc, cfg, layers, g, caches, pos, tok)
        got, nxt = d.forward_token(tok)
        err = rel_rms_err(got, want)
        assert err < DECODER_TOL, (pos, err)
        assert nxt == orc.argmax(got)
    assert d.kernels_per_token() > 0
    # greedy feedback on the device equals feeding the arg-max back from the host
    d.set_position(0)
    toks, ms = d.generate(first_token=42, n_tokens=5)
    d.set_position(0)
    cur, seq = 42, []
    for _ in range(5):
        _, cur = d.forward_token(cur)
        seq.append(cur)
    assert list(toks) == seq and ms > 0
    d.close()


def test_typed_engine_with_default_types_is_the_default_engine(orc):
    """All projections Q4_K, half embedding and head: the typed constructor builds the engine
    mg_decoder_create builds, bit for bit."""
    cfg, seed = SMALL, 43
    a = dec.Q4KDecoder(cfg, types=([[Q4] * 7] * cfg.n_layers, F16, F16))
    b = dec.Q4KDecoder(cfg)
    a.load_random(seed)
    b.load_random(seed)
    assert a.kernels_per_token() == b.kernels_per_token()
    for tok in (5, 639):
        la, na = a.forward_token(tok)
        lb, nb = b.forward_token(tok)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)) and na == nb
    a.close()
    b.close()


def test_typed_engine_refuses_types_without_a_kernel():
    cfg = SMALL
    bad = [[Q4] * 7 for _ in range(cfg.n_layers)]
    bad[1][2] = 8    # Q8_0
    with pytest.raises(Runtime):
        dec.Q4KDecoder(cfg, types=(bad, F16, F16))
    with pytest.raises(Runtime):
        dec.Q4KDecoder(cfg, types=([[Q4] * 7] * cfg.n_layers, 0, F16))   # f32 embedding
    d = dec.Q4KDecoder(cfg, types=(MIX, Q6, Q6))
    with pytest.raises(Runtime, match="size mismatch"):   # Q4_K bytes where the engine holds a Q6_K tensor
        d.upload(0, dec.W_V, synth.q4k_matrix(cfg.kv_dim, cfg.d_model, 1))
    d.close()


@pytest.mark.parametrize("tied", [False, True])
def test_mixed_gguf_loads_into_the_typed_engine(orc, tmp_path, tied):
    cfg, seed = SMALL, 45
    layers, g = mixed_model(cfg, seed, MIX, Q6, Q6)
    if tied:
        g["lm_head"] = g["embed"]
    path = tmp_path / "mixed.gguf"
    path.write_bytes(gw.decoder_gguf(cfg, layers, g, tied=tied))
    a = dec.Q4KDecoder.from_gguf(path, cfg.max_seq)
    assert a.weight_type(0, dec.W_DOWN) == Q6 and a.weight_type(0, dec.W_K) == Q5 and a.weight_type(0, dec.W_LM_HEAD) == Q6
    b = dec.Q4KDecoder(cfg, types=(MIX, Q6, Q6))
    upload_model(b, cfg, layers, g)
    caches = [(np.zeros(cfg.max_seq * cfg.kv_dim, dtype=np.float16), np.zeros(cfg.max_seq * cfg.kv_dim, dtype=np.float16))
              for _ in range(cfg.n_layers)]
    for pos, tok in enumerate((5, 639, 17)):
        la, na = a.forward_token(tok)
        lb, nb = b.forward_token(tok)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)) and na == nb
        assert rel_rms_err(la, oracle_forward(orc, cfg, layers, g, caches, pos, tok)) < DECODER_TOL
    base, nbytes = a.weight_arena()
    for l in range(cfg.n_layers):
        for which in range(9):
            assert base <= a.weight_ptr(l, which) < base + nbytes and a.weight_ptr(l, which) % 256 == 0
    a.close()
    b.close()

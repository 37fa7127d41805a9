"""GGUF checkpoint -> device engine (mg_decoder_load_gguf): a writer in tests/ emits a small GGUF v3
file from synthetic tensors; the loaded engine must produce the same logits, bit for bit, as the
engine fed the same host tensors through mg_decoder_upload, keep every weight in ONE allocation,
refuse what it cannot run and respect the VRAM guard (crates/modgrad-gemma/src/rocm_gemma.rs:94-262)."""
import numpy as np
import pytest

import gguf_writer as gw
from modgrad_b200 import decoder as dec
from modgrad_b200.backend import OutOfMemory, Runtime

pytestmark = pytest.mark.gpu

SMALL = dec.DecoderConfig(n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, d_ff=1024, vocab=640,
                          max_seq=40, rms_eps=1e-6, rope_base=1e6)


def host_model(cfg, seed):
    return [dec.layer_weights(cfg, l, seed) for l in range(cfg.n_layers)], dec.global_weights(cfg, seed)


@pytest.mark.parametrize("tied", [False, True])
def test_loaded_engine_equals_uploaded_engine_bit_for_bit(tmp_path, tied):
    cfg, seed = SMALL, 21
    layers, g = host_model(cfg, seed)
    path = tmp_path / "model.gguf"
    path.write_bytes(gw.decoder_gguf(cfg, layers, g, tied=tied))
    a = dec.Q4KDecoder.from_gguf(path, cfg.max_seq)
    assert (a.cfg.n_layers, a.cfg.d_model, a.cfg.n_heads, a.cfg.n_kv_heads, a.cfg.head_dim, a.cfg.d_ff, a.cfg.vocab) == \
           (2, 512, 4, 2, 128, 1024, 640)
    assert a.cfg.rope_base == np.float32(1e6) and a.cfg.rms_eps == np.float32(1e-6)
    b = dec.Q4KDecoder(cfg)
    b.load_random(seed)
    if tied:
        b.upload(0, dec.W_LM_HEAD, g["embed"])
    for tok in (5, 639, 17):
        la, na = a.forward_token(tok)
        lb, nb = b.forward_token(tok)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)) and na == nb
    # one allocation holds every tensor
    base, nbytes = a.weight_arena()
    assert base and nbytes >= sum(cfg.q4k_bytes_per_layer() for _ in range(cfg.n_layers))
    for l in range(cfg.n_layers):
        for which in range(9):
            p = a.weight_ptr(l, which)
            assert base <= p < base + nbytes and p % 256 == 0
    for which in (dec.W_EMBED, dec.W_LM_HEAD, dec.W_OUT_NORM):
        assert base <= a.weight_ptr(0, which) < base + nbytes
    a.close()
    b.close()


def test_loader_refuses_what_it_cannot_run(tmp_path):
    cfg, seed = SMALL, 22
    layers, g = host_model(cfg, seed)
    good = gw.decoder_gguf(cfg, layers, g)
    # truncated: tensor data runs past the end of the file
    p = tmp_path / "cut.gguf"
    p.write_bytes(good[: len(good) - 100_000])
    with pytest.raises(Runtime, match="past the end"):
        dec.Q4KDecoder.from_gguf(p, cfg.max_seq)
    # a projection in a type the engine has no kernel for (F16 where Q4_K is expected)
    bad_layers = [dict(l) for l in layers]
    blob = gw.decoder_gguf(cfg, bad_layers, g)
    at = blob.index(b"blk.1.ffn_up.weight") + len(b"blk.1.ffn_up.weight") + 4 + 16
    blob = blob[:at] + (1).to_bytes(4, "little") + blob[at + 4:]
    p = tmp_path / "f16.gguf"
    p.write_bytes(blob)
    with pytest.raises(Runtime, match="ffn_up.weight: tensor type 1"):
        dec.Q4KDecoder.from_gguf(p, cfg.max_seq)
    # a missing tensor and a missing metadata key
    p = tmp_path / "missing.gguf"
    p.write_bytes(good.replace(b"blk.0.attn_v.weight", b"blk.0.attn_x.weight"))
    with pytest.raises(Runtime, match="missing blk.0.attn_v.weight"):
        dec.Q4KDecoder.from_gguf(p, cfg.max_seq)
    p = tmp_path / "nokey.gguf"
    p.write_bytes(good.replace(b"qwen2.block_count", b"qwen2.block_coumt"))
    with pytest.raises(Runtime, match="missing qwen2.block_count"):
        dec.Q4KDecoder.from_gguf(p, cfg.max_seq)
    with pytest.raises(Runtime, match="cannot open"):
        dec.Q4KDecoder.from_gguf(tmp_path / "nope.gguf", cfg.max_seq)


def test_vram_guard_refuses_to_over_commit(tmp_path, monkeypatch):
    cfg, seed = SMALL, 23
    layers, g = host_model(cfg, seed)
    p = tmp_path / "m.gguf"
    p.write_bytes(gw.decoder_gguf(cfg, layers, g))
    monkeypatch.setenv("MODGRAD_VRAM_MARGIN_MB", str(1 << 20))   # a margin no device has
    with pytest.raises(OutOfMemory, match="over-commit VRAM"):
        dec.Q4KDecoder.from_gguf(p, cfg.max_seq)
    monkeypatch.delenv("MODGRAD_VRAM_MARGIN_MB")
    d = dec.Q4KDecoder.from_gguf(p, cfg.max_seq)
    d.close()

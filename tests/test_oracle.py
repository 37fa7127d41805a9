"""CPU tests: the oracle against the hand-built known-answer blocks and against an
independent numpy restatement; the seeded generator; host-side properties."""
import hashlib

import numpy as np
import pytest

from conftest import GEMV_TOL, rel_rms_err
from modgrad_b200 import synth
from oracle import q4k_numpy as qn
from oracle.loader import MODE_F64, MODE_SCALAR, MODE_SELECT


def test_kats_dequant_bit_exact_c_and_numpy(orc, kats):
    for k in kats:
        got_c = orc.dequantize(k["block"])
        got_np = qn.dequantize(k["block"]).reshape(-1)
        assert np.array_equal(got_c.view(np.uint32), k["expected"].view(np.uint32)), k["name"]
        assert np.array_equal(got_np.view(np.uint32), k["expected"].view(np.uint32)), k["name"]


def test_kats_scale_unpack(orc, kats):
    for k in kats:
        if "sc" not in k:
            continue
        scales = k["block"][4:16]
        sc_np, m_np = qn.scale_min_k4(scales)
        for j in range(8):
            assert orc.get_scale_min_k4(j, scales) == (k["sc"][j], k["m"][j])
        assert list(sc_np) == k["sc"] and list(m_np) == k["m"]
        # the packer is the inverse
        assert np.array_equal(qn.pack_scales_mins(np.array(k["sc"]), np.array(k["m"])), scales)
        assert np.array_equal(synth.pack_scales_mins(np.array([k["sc"]]), np.array([k["m"]]))[0], scales)


def test_kats_matvec_known_answers(orc, kats):
    for k in kats:
        x = np.array(k["x_ramp"], dtype=np.float32)
        want = k["y_ramp"][0] / k["y_ramp"][1]
        for mode in (MODE_SCALAR, MODE_SELECT, MODE_F64):
            y = orc.matvec(k["block"], x, 1, 1, mode)[0]
            assert abs(float(y) - want) <= 1e-5 * max(1.0, abs(want)), (k["name"], mode)
        # element order pinned independently of any sum: a one-hot x picks one weight
        for e in (0, 31, 32, 63, 64, 100, 255):
            onehot = np.zeros(256, dtype=np.float32)
            onehot[e] = 1.0
            y = orc.matvec(k["block"], onehot, 1, 1, MODE_SCALAR)[0]
            exp = k["expected"][e]
            assert y == exp or (y == 0 and exp == 0), (k["name"], e)


def test_f16_decode_all_patterns(orc):
    h = np.arange(65536, dtype=np.uint16)
    want = qn.f16_to_f32(h)
    got = np.array([orc.f16_to_f32(int(v)) for v in h], dtype=np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))
    # exponent 31 covers inf and NaN: both NaN, as the reference decodes them
    assert np.isnan(got[0x7C00]) and np.isnan(got[0xFC00]) and np.isnan(got[0x7E00])


def test_c_oracle_equals_numpy_on_random_blocks(orc):
    rng = np.random.Generator(np.random.PCG64(7))
    blocks = synth.q4k_blocks(512, rng)
    # sprinkle special scales: inf, NaN, sub-normal, negative
    specials = [0x7C00, 0xFC00, 0x7E00, 0x0001, 0x83FF, 0x8000, 0x0000, 0x7BFF, 0xBC00]
    for i, s in enumerate(specials):
        blocks[i, 0:2] = [s & 0xFF, s >> 8]
        blocks[-1 - i, 2:4] = [s & 0xFF, s >> 8]
    a = orc.dequantize(blocks)
    b = qn.dequantize(blocks).reshape(-1)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert np.all(np.isfinite(a))


def test_dequant_is_pure_function_of_bytes(orc):
    # crates/modgrad-device/src/kfd/gguf.rs:745-760
    blocks = synth.q4k_blocks(2, np.random.Generator(np.random.PCG64(1)))
    assert np.array_equal(orc.dequantize(blocks).view(np.uint32), orc.dequantize(blocks.copy()).view(np.uint32))


@pytest.mark.parametrize("out_dim,bpr", [(1, 1), (3, 2), (64, 4), (33, 5), (8, 74)])
def test_matvec_modes_agree(orc, out_dim, bpr):
    w = synth.q4k_matrix(out_dim, bpr * 256, 11)
    x = synth.activations(bpr * 256, 12)
    y64 = orc.matvec_f64(w, x, out_dim, bpr)
    ynp = qn.matvec_f64(w.reshape(-1, 144), x, out_dim, bpr)
    assert np.allclose(y64, ynp, rtol=1e-12, atol=1e-9)
    for mode in (MODE_SCALAR, MODE_SELECT, MODE_F64):
        y = orc.matvec(w, x, out_dim, bpr, mode)
        # the reference's own f32 arms are reorderings of the same sum
        assert rel_rms_err(y, y64) < 5e-5
    # row partition over threads does not change any row
    y1 = orc.matvec(w, x, out_dim, bpr, MODE_SCALAR, threads=1)
    y8 = orc.matvec(w, x, out_dim, bpr, MODE_SCALAR, threads=8)
    assert np.array_equal(y1.view(np.uint32), y8.view(np.uint32))


def test_matvec_is_dequant_times_x(orc):
    out_dim, bpr = 16, 3
    w = synth.q4k_matrix(out_dim, bpr * 256, 21)
    x = synth.activations(bpr * 256, 22)
    dq = orc.dequantize(w).reshape(out_dim, bpr * 256).astype(np.float64)
    assert np.allclose(dq @ x.astype(np.float64), orc.matvec_f64(w, x, out_dim, bpr), rtol=1e-13, atol=1e-10)


def test_config0_generator_is_pinned(orc):
    """Regression pins of THIS repository's generator and oracle (not reference vectors):
    a changed PRNG stream or a changed oracle shows up here before any GPU run."""
    rng = np.random.Generator(np.random.PCG64(42))
    w = synth.q4k_matrix(64, 4096, rng)          # first 64 rows of the 4096 x 4096 case
    x = synth.activations(4096, rng)
    assert w.size == 64 * 16 * 144
    assert hashlib.sha256(w.tobytes()).hexdigest()[:16] == PIN_W
    assert hashlib.sha256(x.tobytes()).hexdigest()[:16] == PIN_X
    y = orc.matvec(w, x, 64, 16, MODE_F64)
    assert hashlib.sha256(y.tobytes()).hexdigest()[:16] == PIN_Y
    # value distributions of the synthetic blocks
    blk = w.reshape(-1, 144)
    d = blk[:, 0:2].copy().view(np.float16)[:, 0].astype(np.float32)
    assert 0 <= d.min() and d.max() < 0.06 and 0.006 < d.mean() < 0.010
    sc, m = qn.scale_min_k4(blk[:, 4:16])
    assert sc.max() == 63 and m.max() == 63 and sc.min() == 0


PIN_W = "1ca9b88b89a70d78"
PIN_X = "3047654ac96a4f04"
PIN_Y = "2e7297e1d2a7b393"


def test_q8_1_side_path_matches_f32_within_band(orc):
    """int8-activation variant: ~1 % class error by design
    (crates/modgrad-device/examples/rocm_dp4a_check.rs:63-65 gates RMS-rel < 2 %)."""
    out_dim, bpr = 32, 4
    w = synth.q4k_matrix(out_dim, bpr * 256, 31)
    x = synth.activations(bpr * 256, 32)
    xq, xd, xs = orc.quantize_q8_1(x)
    assert np.all(np.abs(xq.astype(np.int32)) <= 127)
    assert np.array_equal(xs, xq.reshape(-1, 32).astype(np.int32).sum(1).astype(np.float32))
    y = orc.matvec_q8_1(w, xq, xd, xs, out_dim, bpr)
    y64 = orc.matvec_f64(w, x, out_dim, bpr)
    assert np.sqrt(np.mean((y - y64) ** 2)) / np.sqrt(np.mean(y64 ** 2)) < 0.02


def test_gemv_bytes_formula():
    assert synth.gemv_bytes(4096, 4096) == 9_469_952
    assert sum(o * (i // 256) * 144 for o, i in synth.QWEN25_7B_LAYER.values()) == 131_088_384
    assert sum(o * (i // 256) * 144 for o, i in synth.LLAMA_70B_LAYER.values()) == 481_296_384


def test_tolerance_constant():
    assert GEMV_TOL == 1e-5


def test_kquant_oracle_matches_kats_and_numpy(orc):
    """Q5_K / Q6_K: the C restatement against the format-derived known-answer blocks (bit-exact)
    and against the independent numpy restatement on random blocks and special scales."""
    import json
    from conftest import GOLDEN
    from oracle import q4k_numpy as qn
    for k in json.loads((GOLDEN / "kquant_kats.json").read_text())["kats"]:
        blk = np.frombuffer(bytes.fromhex(k["block_hex"]), dtype=np.uint8)
        want = np.array(k["expected_f32_bits"], dtype=np.uint32)
        assert np.array_equal(orc.dequantize_kquant(k["kind"], blk).view(np.uint32), want), k["name"]
    rng = np.random.Generator(np.random.PCG64(12))
    for kind, gen, fn in ((5, synth.q5k_blocks, qn.dequantize_q5k), (6, synth.q6k_blocks, qn.dequantize_q6k)):
        b = gen(3000, rng)
        off = 0 if kind == 5 else 208
        b[0, off:off + 2], b[1, off:off + 2], b[2, off:off + 2] = [0, 0x7C], [1, 0x7E], [1, 0]
        assert np.array_equal(orc.dequantize_kquant(kind, b).view(np.uint32), fn(b).view(np.uint32))
        w = gen(4 * 3, rng).reshape(-1)
        x = synth.activations(3 * 256, rng)
        y = orc.matvec_kquant_f64(kind, w, x, 4, 3)
        ref = fn(w).reshape(4, -1).astype(np.float64) @ x.astype(np.float64)
        assert np.allclose(y, ref, rtol=1e-12, atol=1e-12)

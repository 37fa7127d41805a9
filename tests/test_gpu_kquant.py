"""GPU parity of the Q5_K and Q6_K kernels through the C ABI against the oracle's restatement of
crates/modgrad-device/src/kfd/gguf.rs:421-484 (dequantised weights: bit-exact, incl. the known-answer
blocks of tests/golden/kquant_kats.json; matvec: 1e-5 of the output RMS against the f64 dot)."""
import json

import numpy as np
import pytest

from conftest import GEMV_TOL, GOLDEN, rel_rms_err, rms
from modgrad_b200 import synth
from modgrad_b200.backend import DeviceBuffer, kern

pytestmark = pytest.mark.gpu
BB = {5: 176, 6: 210}


def upload(a):
    a = np.ascontiguousarray(a)
    b = DeviceBuffer(a.nbytes)
    b.copy_from_host_bytes(a)
    return b


def gpu_dequant(cuda, kind, blocks):
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    n = blocks.size // BB[kind]
    src, dst = upload(blocks), DeviceBuffer(n * 1024)
    fn = cuda.mg_dequant_q5k_on_stream if kind == 5 else cuda.mg_dequant_q6k_on_stream
    assert fn(src.ptr, n, dst.ptr, None) == 0
    kern.sync()
    return dst.copy_to_host(n * 256)


def gpu_matvec(cuda, kind, w, x, out_dim, bpr):
    wd, xd, yd = upload(w), upload(x), DeviceBuffer(out_dim * 4)
    fn = cuda.launch_matvec_q5k if kind == 5 else cuda.launch_matvec_q6k
    assert fn(wd.ptr, xd.ptr, yd.ptr, out_dim, bpr) == 0
    kern.sync()
    return yd.copy_to_host(out_dim)


def test_kquant_kats_bit_exact(cuda):
    for k in json.loads((GOLDEN / "kquant_kats.json").read_text())["kats"]:
        blk = np.frombuffer(bytes.fromhex(k["block_hex"]), dtype=np.uint8)
        want = np.array(k["expected_f32_bits"], dtype=np.uint32)
        assert np.array_equal(gpu_dequant(cuda, k["kind"], blk).view(np.uint32), want), k["name"]
        x = np.array(k["x_ramp"], dtype=np.float32)
        y = gpu_matvec(cuda, k["kind"], blk, x, 1, 1)[0]
        ref = k["y_ramp"][0] / k["y_ramp"][1]
        assert abs(float(y) - ref) <= 1e-5 * max(1.0, abs(ref)), k["name"]


@pytest.mark.parametrize("kind", [5, 6])
@pytest.mark.parametrize("n_blocks", [1, 8, 1000, 65536])
def test_kquant_dequant_random_blocks_bit_exact(orc, cuda, kind, n_blocks):
    rng = np.random.Generator(np.random.PCG64(300 + n_blocks + kind))
    blocks = (synth.q5k_blocks if kind == 5 else synth.q6k_blocks)(n_blocks, rng)
    off = 0 if kind == 5 else 208
    if n_blocks >= 8:   # non-finite, sub-normal and negative-zero super-block scales
        blocks[0, off:off + 2] = [0x00, 0x7C]
        blocks[1, off:off + 2] = [0x01, 0xFE]
        blocks[2, off:off + 2] = [0x01, 0x00]
        blocks[3, off:off + 2] = [0x00, 0x80]
    got, want = gpu_dequant(cuda, kind, blocks), orc.dequantize_kquant(kind, blocks)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("kind", [5, 6])
@pytest.mark.parametrize("out_dim,bpr", [(1, 1), (7, 3), (513, 14), (3584, 74), (4096, 16), (9000, 14), (100, 40),
                                         (5000, 33), (149, 264)])
def test_kquant_matvec(orc, cuda, kind, out_dim, bpr):
    rng = np.random.Generator(np.random.PCG64(400 + out_dim + bpr + kind))
    w = synth.kquant_matrix(kind, out_dim, bpr * 256, rng)
    x = synth.activations(bpr * 256, rng)
    y = gpu_matvec(cuda, kind, w, x, out_dim, bpr)
    assert rel_rms_err(y, orc.matvec_kquant_f64(kind, w, x, out_dim, bpr)) <= GEMV_TOL


@pytest.mark.parametrize("kind,out_dim,bpr,x_kind", [(6, 3584, 74, 1), (6, 3585, 14, 1), (6, 33, 3, 1), (6, 3584, 74, 0),
                                                     (6, 640, 14, 0), (5, 3584, 74, 0), (5, 129, 14, 0), (5, 3584, 74, 1),
                                                     (5, 3585, 14, 1), (5, 33, 3, 1), (5, 152064, 2, 1)])
def test_kquant_matvec_with_residual_and_limb_records(orc, cuda, kind, out_dim, bpr, x_kind):
    """mg_matvec_kquant_on_stream: y = add + W x in place, from f32 activations or from limb records."""
    rng = np.random.Generator(np.random.PCG64(900 + out_dim + bpr + kind + x_kind))
    k = bpr * 256
    w = synth.kquant_matrix(kind, out_dim, k, rng)
    x = synth.activations(k, rng)
    add = synth.activations(out_dim, rng) * np.float32(3.0)
    wd, xd, yd = upload(w), upload(x), upload(add)
    src = xd
    if x_kind == 1:
        src = DeviceBuffer(cuda.mg_q4k_limb_record_bytes(k))
        assert cuda.mg_q4k_x_to_limbs_on_stream(xd.ptr, k, src.ptr, None) == 0
    assert cuda.mg_matvec_kquant_on_stream(8 + kind, wd.ptr, src.ptr, x_kind, yd.ptr, yd.ptr, out_dim, bpr, None) == 0
    kern.sync()
    want = orc.matvec_kquant_f64(kind, w, x, out_dim, bpr)
    got = yd.copy_to_host(out_dim).astype(np.float64) - add.astype(np.float64)
    assert rms(got - want) / rms(want) <= GEMV_TOL
    # without the addend
    y2 = DeviceBuffer(out_dim * 4)
    assert cuda.mg_matvec_kquant_on_stream(8 + kind, wd.ptr, src.ptr, x_kind, None, y2.ptr, out_dim, bpr, None) == 0
    kern.sync()
    assert rel_rms_err(y2.copy_to_host(out_dim), want) <= GEMV_TOL


@pytest.mark.parametrize("kind,out_dim,bpr", [(6, 512, 14), (5, 512, 14), (6, 9000, 14), (5, 4099, 2), (6, 300, 40)])
def test_rmsnorm_fused_in_front_of_kquant_matvec(orc, cuda, kind, out_dim, bpr):
    """y = W . rms_norm(x): the norm of crates/modgrad-device/src/kfd/llm.rs:921-928 done by every CTA while it
    converts x, against the oracle's rms_norm followed by its f64 matvec."""
    rng = np.random.Generator(np.random.PCG64(950 + out_dim + bpr + kind))
    k = bpr * 256
    w = synth.kquant_matrix(kind, out_dim, k, rng)
    x = synth.activations(k, rng) * np.float32(3.0)
    nw = (1.0 + 0.05 * rng.standard_normal(k, dtype=np.float32)).astype(np.float32)
    eps = 1e-6
    wd, xd, nd, yd = upload(w), upload(x), upload(nw), DeviceBuffer(out_dim * 4)
    assert cuda.mg_rmsnorm_matvec_kquant_on_stream(8 + kind, wd.ptr, xd.ptr, nd.ptr, eps, yd.ptr, out_dim, bpr, None) == 0
    kern.sync()
    want = orc.matvec_kquant_f64(kind, w, orc.rms_norm(x, nw, eps), out_dim, bpr)
    assert rel_rms_err(yd.copy_to_host(out_dim), want) <= 2 * GEMV_TOL   # the norm's own f32 rounding rides on top
    assert cuda.mg_rmsnorm_matvec_kquant_on_stream(8 + kind, wd.ptr, xd.ptr, None, eps, yd.ptr, out_dim, bpr, None) == 1
    assert cuda.mg_rmsnorm_matvec_kquant_on_stream(12, wd.ptr, xd.ptr, nd.ptr, eps, yd.ptr, out_dim, bpr, None) == 1


def test_q6k_weight_that_is_only_two_byte_aligned(orc, cuda):
    """Q6_K rows are 2-byte aligned; a weight that starts 2 bytes into a word takes the float kernel and refuses records."""
    out_dim, bpr = 300, 14
    rng = np.random.Generator(np.random.PCG64(93))
    w = synth.kquant_matrix(6, out_dim, bpr * 256, rng)
    x = synth.activations(bpr * 256, rng)
    buf = DeviceBuffer(w.nbytes + 16)
    shifted = np.concatenate([np.zeros(2, dtype=np.uint8), w, np.zeros(14, dtype=np.uint8)])
    buf.copy_from_host_bytes(shifted)
    xd, yd = upload(x), DeviceBuffer(out_dim * 4)
    assert cuda.launch_matvec_q6k(buf.ptr + 2, xd.ptr, yd.ptr, out_dim, bpr) == 0
    kern.sync()
    assert rel_rms_err(yd.copy_to_host(out_dim), orc.matvec_kquant_f64(6, w, x, out_dim, bpr)) <= GEMV_TOL
    rec = DeviceBuffer(cuda.mg_q4k_limb_record_bytes(bpr * 256))
    assert cuda.mg_q4k_x_to_limbs_on_stream(xd.ptr, bpr * 256, rec.ptr, None) == 0
    assert cuda.mg_matvec_kquant_on_stream(14, buf.ptr + 2, rec.ptr, 1, None, yd.ptr, out_dim, bpr, None) == 1
    assert cuda.mg_matvec_kquant_on_stream(12, buf.ptr, xd.ptr, 0, None, yd.ptr, out_dim, bpr, None) == 1
    kern.sync()


@pytest.mark.parametrize("kind", [5, 6])
def test_kquant_non_finite_activation_poisons_every_row(cuda, kind):
    out_dim, bpr = 64, 14
    rng = np.random.Generator(np.random.PCG64(94))
    w = synth.kquant_matrix(kind, out_dim, bpr * 256, rng)
    x = synth.activations(bpr * 256, rng)
    x[1000] = np.inf
    y = gpu_matvec(cuda, kind, w, x, out_dim, bpr)
    assert np.all(np.isnan(y))


def test_kquant_matvec_equals_dequant_then_dot(cuda):
    for kind in (5, 6):
        out_dim, bpr = 96, 5
        rng = np.random.Generator(np.random.PCG64(77 + kind))
        w = synth.kquant_matrix(kind, out_dim, bpr * 256, rng)
        x = synth.activations(bpr * 256, rng)
        dq = gpu_dequant(cuda, kind, w).reshape(out_dim, -1).astype(np.float64)
        assert rel_rms_err(gpu_matvec(cuda, kind, w, x, out_dim, bpr), dq @ x.astype(np.float64)) <= GEMV_TOL


def test_q6k_dp4a_matches_reference_arithmetic(orc, cuda):
    out_dim, bpr = 640, 14
    rng = np.random.Generator(np.random.PCG64(91))
    w = synth.kquant_matrix(6, out_dim, bpr * 256, rng)
    x = synth.activations(bpr * 256, rng)
    n = x.size
    xd_, xq, xd, xs = upload(x), DeviceBuffer(n), DeviceBuffer(n // 8), DeviceBuffer(n // 8)
    kern.quantize_q8_1(xd_.ptr, xq.ptr, xd.ptr, xs.ptr, n)
    wd, yd = upload(w), DeviceBuffer(out_dim * 4)
    assert cuda.launch_matvec_q6k_dp4a(wd.ptr, xq.ptr, xd.ptr, xs.ptr, yd.ptr, out_dim, bpr) == 0
    kern.sync()
    y = yd.copy_to_host(out_dim)
    q = np.empty(n, dtype=np.int8)
    xq.copy_to_host_bytes(q.view(np.uint8))
    want = orc.matvec_q6k_q8_1(w, q, xd.copy_to_host(n // 32), out_dim, bpr)
    assert rel_rms_err(y, want.astype(np.float64)) <= GEMV_TOL
    y64 = orc.matvec_kquant_f64(6, w, x, out_dim, bpr)
    assert rms(y - y64) / rms(y64) < 0.02     # the lossy path against the f32 one


def test_kquant_bad_arguments(cuda):
    b = DeviceBuffer(1024)
    assert cuda.launch_matvec_q5k(b.ptr, b.ptr, b.ptr, 0, 1) == 1
    assert cuda.launch_matvec_q6k(b.ptr, b.ptr, b.ptr, 1, 0) == 1
    assert cuda.launch_matvec_q6k(None, b.ptr, b.ptr, 1, 1) == 1
    assert cuda.launch_matvec_q5k(b.ptr + 8, b.ptr, b.ptr, 1, 1) == 1     # Q5_K rows must be 16-byte aligned

"""GPU parity tests, through the C ABI, against the CPU oracle on identical seeded bytes.

Dequantised weights: bit-exact.  Dot products: max|y - y_ref| / rms(y_ref) <= 1e-5 against
the f64-accumulated oracle (f32 accumulate, reordered sums)."""
import ctypes as C

import numpy as np
import pytest

from conftest import GEMV_TOL, rel_rms_err
from modgrad_b200 import backend, synth
from modgrad_b200.backend import DeviceBuffer, kern
from oracle.loader import MODE_SCALAR, MODE_SELECT

pytestmark = pytest.mark.gpu


def upload(a: np.ndarray) -> DeviceBuffer:
    a = np.ascontiguousarray(a)
    b = DeviceBuffer(a.nbytes)
    b.copy_from_host_bytes(a)
    return b


def gpu_dequant(blocks: np.ndarray) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    n = blocks.size // 144
    src, dst = upload(blocks), DeviceBuffer(n * 1024)
    kern.dequant_q4k(src.ptr, n, dst.ptr)
    kern.sync()
    return dst.copy_to_host(n * 256)


def gpu_matvec(w, x, out_dim, bpr):
    wd, xd, yd = upload(w), upload(x), DeviceBuffer(out_dim * 4)
    kern.matvec_q4k(wd.ptr, xd.ptr, yd.ptr, out_dim, bpr)
    kern.sync()
    return yd.copy_to_host(out_dim)


# ---- dequantisation: bit-exact ----------------------------------------------------------------
def test_dequant_kats_bit_exact(kats):
    for k in kats:
        got = gpu_dequant(k["block"])
        assert np.array_equal(got.view(np.uint32), k["expected"].view(np.uint32)), k["name"]
    allb = np.concatenate([k["block"] for k in kats])
    want = np.concatenate([k["expected"] for k in kats])
    assert np.array_equal(gpu_dequant(allb).view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("n_blocks", [1, 8, 9, 1000, 4096 * 16])
def test_dequant_random_blocks_bit_exact(orc, n_blocks):
    # n_blocks 1 and 8 are the reference's own cases (crates/modgrad-device/tests/dequant_q4k.rs:49-130)
    blocks = synth.q4k_blocks(n_blocks, np.random.Generator(np.random.PCG64(100 + n_blocks)))
    assert np.array_equal(gpu_dequant(blocks).view(np.uint32), orc.dequantize(blocks).view(np.uint32))


def test_dequant_every_half_pattern_bit_exact(orc):
    """All 65536 bit patterns of d and of dmin: finite, sub-normal, inf, NaN, signed zero."""
    rng = np.random.Generator(np.random.PCG64(5))
    blocks = synth.q4k_blocks(2 * 65536, rng)
    h = np.arange(65536, dtype=np.uint16)
    blocks[:65536, 0:2] = h.view(np.uint8).reshape(-1, 2)
    blocks[65536:, 2:4] = h.view(np.uint8).reshape(-1, 2)
    got, want = gpu_dequant(blocks), orc.dequantize(blocks)
    assert np.all(np.isfinite(got))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequant_is_pure_function_of_bytes():
    blocks = synth.q4k_blocks(64, np.random.Generator(np.random.PCG64(3)))
    a, b = gpu_dequant(blocks), gpu_dequant(blocks.copy())
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


# ---- matvec -------------------------------------------------------------------------------------
def check_matvec(orc, out_dim, bpr, seed, tol=GEMV_TOL):
    rng = np.random.Generator(np.random.PCG64(seed))
    w = synth.q4k_matrix(out_dim, bpr * 256, rng)
    x = synth.activations(bpr * 256, rng)
    y = gpu_matvec(w, x, out_dim, bpr)
    y64 = orc.matvec_f64(w, x, out_dim, bpr)
    err = rel_rms_err(y, y64)
    assert err <= tol, f"{out_dim}x{bpr * 256}: {err:.3e} > {tol}"
    return w, x, y, y64


def test_matvec_config0(orc):
    """4096 x 4096, seed 42: the reference's CPU-runnable case."""
    w, x, y, y64 = check_matvec(orc, 4096, 16, 42)
    # beside it: distance to the reference's own f32 arms (reorderings of the same sum)
    for mode in (MODE_SCALAR, MODE_SELECT):
        assert rel_rms_err(y, orc.matvec(w, x, 4096, 16, mode).astype(np.float64)) < 5e-5


@pytest.mark.parametrize("name", list(synth.QWEN25_7B_LAYER))
def test_matvec_qwen7b_layer_shapes(orc, name):
    out_dim, in_dim = synth.QWEN25_7B_LAYER[name]
    check_matvec(orc, out_dim, in_dim // 256, 1000 + len(name))


@pytest.mark.parametrize("out_dim,bpr", [(1, 1), (2, 1), (7, 3), (33, 5), (257, 2), (8, 113), (5, 130),
                                         (1184, 14), (1185, 14), (2369, 4), (100, 74)])
def test_matvec_ragged_shapes(orc, out_dim, bpr):
    check_matvec(orc, out_dim, bpr, 7000 + out_dim * 131 + bpr)


@pytest.mark.parametrize("name", list(synth.LLAMA_70B_LAYER))
def test_matvec_llama70b_layer_shapes(orc, name):
    """The 70B-class projections (rows of 8192 and 28672 weights: 32 and 112 super-blocks)."""
    out_dim, in_dim = synth.LLAMA_70B_LAYER[name]
    check_matvec(orc, out_dim, in_dim // 256, 2000 + len(name))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_matvec_llama70b_per_rank_slices(orc, world):
    """What one rank of a row-sharded 70B-class layer computes: a contiguous row range of the
    unmodified block array (k_proj and down_proj: the smallest and the longest-row slices)."""
    for name in ("k_proj", "down_proj"):
        out_dim, in_dim = synth.LLAMA_70B_LAYER[name]
        bpr, rows = in_dim // 256, out_dim // world
        rng = np.random.Generator(np.random.PCG64(3000 + world))
        w = synth.q4k_matrix(rows, in_dim, rng)
        x = synth.activations(in_dim, rng)
        assert rel_rms_err(gpu_matvec(w, x, rows, bpr), orc.matvec_f64(w, x, rows, bpr)) <= GEMV_TOL


def test_matvec_kats(kats):
    for k in kats:
        x = np.array(k["x_ramp"], dtype=np.float32)
        want = k["y_ramp"][0] / k["y_ramp"][1]
        y = gpu_matvec(k["block"], x, 1, 1)[0]
        assert abs(float(y) - want) <= 1e-5 * max(1.0, abs(want)), k["name"]
        for e in (0, 31, 32, 63, 64, 100, 255):  # element order, independent of any sum
            onehot = np.zeros(256, dtype=np.float32)
            onehot[e] = 1.0
            assert gpu_matvec(k["block"], onehot, 1, 1)[0] == k["expected"][e], (k["name"], e)


def test_matvec_nonfinite_block_scales_contribute_zero(orc):
    w = synth.q4k_matrix(16, 1024, 77).reshape(-1, 144)
    w[0, 0:2] = [0x00, 0x7C]   # d = +inf
    w[5, 2:4] = [0x01, 0x7E]   # dmin = NaN
    w[9, 0:4] = [0x00, 0xFC, 0xFF, 0xFF]
    x = synth.activations(1024, 78)
    y = gpu_matvec(w.reshape(-1), x, 16, 4)
    assert np.all(np.isfinite(y))
    assert rel_rms_err(y, orc.matvec_f64(w.reshape(-1), x, 16, 4)) <= GEMV_TOL


def test_matvec_with_bias_and_unaligned_x(orc, cuda):
    out_dim, bpr = 300, 6
    rng = np.random.Generator(np.random.PCG64(9))
    w = synth.q4k_matrix(out_dim, bpr * 256, rng)
    x = synth.activations(bpr * 256, rng)
    bias = synth.activations(out_dim, rng)
    wd, yd, bd = upload(w), DeviceBuffer(out_dim * 4), upload(bias)
    xpad = DeviceBuffer(x.nbytes + 16)
    assert cuda.mg_memcpy_h2d(xpad.ptr + 4, x.ctypes.data_as(C.c_void_p), x.nbytes) == 0
    assert cuda.mg_matvec_q4k_bias_on_stream(wd.ptr, xpad.ptr + 4, bd.ptr, yd.ptr, out_dim, bpr, None) == 0
    kern.sync()
    y64 = orc.matvec_f64(w, x, out_dim, bpr) + bias.astype(np.float64)
    assert rel_rms_err(yd.copy_to_host(out_dim), y64) <= GEMV_TOL


def test_matvec_linearity_at_full_size():
    """Size-independent property on the largest 7B projection: W(a x1 + b x2) = a W x1 + b W x2."""
    out_dim, in_dim = synth.QWEN25_7B_LAYER["gate_proj"]
    rng = np.random.Generator(np.random.PCG64(55))
    w = synth.q4k_matrix(out_dim, in_dim, rng)
    x1, x2 = synth.activations(in_dim, rng), synth.activations(in_dim, rng)
    bpr = in_dim // 256
    y1, y2 = gpu_matvec(w, x1, out_dim, bpr), gpu_matvec(w, x2, out_dim, bpr)
    y12 = gpu_matvec(w, (2.0 * x1 - 0.5 * x2).astype(np.float32), out_dim, bpr)
    want = 2.0 * y1.astype(np.float64) - 0.5 * y2.astype(np.float64)
    assert rel_rms_err(y12, want) <= 4 * GEMV_TOL
    # and a row permutation of W permutes y (rows are independent)
    perm = rng.permutation(out_dim)
    wp = w.reshape(out_dim, -1)[perm].reshape(-1)
    assert np.array_equal(gpu_matvec(wp, x1, out_dim, bpr), y1[perm])


def test_matvec_equals_dequant_then_dot():
    """The fused kernel agrees with the GPU's own bit-exact dequantiser followed by an f64 dot."""
    out_dim, bpr = 512, 14
    rng = np.random.Generator(np.random.PCG64(66))
    w = synth.q4k_matrix(out_dim, bpr * 256, rng)
    x = synth.activations(bpr * 256, rng)
    dq = gpu_dequant(w).reshape(out_dim, bpr * 256).astype(np.float64)
    assert rel_rms_err(gpu_matvec(w, x, out_dim, bpr), dq @ x.astype(np.float64)) <= GEMV_TOL


# ---- operator / plugin tier ---------------------------------------------------------------------
def test_backend_matvec_op_host_slices(orc):
    be = backend.CudaBackend.try_new(0)
    assert be is not None and be.name() == "cuda" and "SMs" in be.device_info()
    out_dim, in_dim = 640, 2048
    rng = np.random.Generator(np.random.PCG64(13))
    w = synth.q4k_matrix(out_dim, in_dim, rng)
    x = synth.activations(in_dim, rng)
    bias = synth.activations(out_dim, rng)
    out = np.zeros(out_dim, dtype=np.float32)
    op = backend.Matvec(x, w, bias, out, out_dim, in_dim, backend.QuantKind.Q4K)
    assert be.supports(op)
    be.dispatch(op)
    y64 = orc.matvec_f64(w, x, out_dim, in_dim // 256)
    assert rel_rms_err(out, y64 + bias) <= GEMV_TOL
    assert be.cached_weights() == 1
    # no bias = empty slice; weights stay resident between dispatches
    out2 = np.zeros(out_dim, dtype=np.float32)
    be.dispatch(backend.Matvec(x, w, np.empty(0, np.float32), out2, out_dim, in_dim, backend.QuantKind.Q4K))
    assert rel_rms_err(out2, y64) <= GEMV_TOL and be.cached_weights() == 1
    be.invalidate_cache()
    assert be.cached_weights() == 0
    # what the backend does not claim
    assert not be.supports(backend.Matvec(x, w, bias, out, out_dim, in_dim, backend.QuantKind.F32))
    assert not be.supports(backend.Matvec(x, w, bias, out, out_dim, in_dim - 1, backend.QuantKind.Q4K))
    assert not be.supports(backend.Matvec(x, w[:-144], bias, out, out_dim, in_dim, backend.QuantKind.Q4K))
    with pytest.raises(backend.Unsupported):
        be.dispatch(backend.Matvec(x, w, bias, out, out_dim, in_dim, backend.QuantKind.F32))


def test_backend_dequant_resident_op(orc):
    # crates/modgrad-device/tests/dequant_q4k.rs:49-130: upload -> Op::DequantQ4KResident -> compare
    for n_blocks in (1, 8):
        blocks = synth.q4k_blocks(n_blocks, np.random.Generator(np.random.PCG64(n_blocks)))
        src, dst = upload(blocks), DeviceBuffer(n_blocks * 1024)
        backend.ops.dequant_q4k_resident(src.ptr, dst.ptr, n_blocks)
        assert np.array_equal(dst.copy_to_host(n_blocks * 256).view(np.uint32),
                              orc.dequantize(blocks).view(np.uint32))
    with pytest.raises(backend.Unsupported):
        backend.ops.dequant_q4k_resident(0, 0, 1)


def test_device_buffer_matvec_host_in_host_out(orc):
    out_dim, bpr = 3584, 14
    rng = np.random.Generator(np.random.PCG64(21))
    w = synth.q4k_matrix(out_dim, bpr * 256, rng)
    x = synth.activations(bpr * 256, rng)
    wd = upload(w)
    y = wd.matvec_q4k(x, out_dim, bpr)
    y64 = orc.matvec_f64(w, x, out_dim, bpr)
    assert rel_rms_err(y, y64) <= GEMV_TOL
    xd, yd = upload(x), DeviceBuffer(out_dim * 4)
    wd.matvec_q4k_into(xd, yd, out_dim, bpr)
    assert np.array_equal(yd.copy_to_host(out_dim), y)
    with pytest.raises(backend.Runtime):
        DeviceBuffer(16).copy_from_host_bytes(np.zeros(32, np.uint8))
    with pytest.raises(backend.Runtime):
        wd.matvec_q4k(x, out_dim + 1, bpr)  # weight buffer too small for the claimed shape


def test_limb_records_two_step_matvec(orc, cuda):
    """Convert x once, run several matvecs on the records (q/k/v and gate/up share their x)."""
    in_dim = 3584
    rng = np.random.Generator(np.random.PCG64(88))
    x = synth.activations(in_dim, rng)
    xd = upload(x)
    nbytes = cuda.mg_q4k_limb_record_bytes(in_dim)
    assert nbytes == (in_dim // 64) * 208
    rec = DeviceBuffer(nbytes)
    assert cuda.mg_q4k_x_to_limbs_on_stream(xd.ptr, in_dim, rec.ptr, None) == 0
    for out_dim in (512, 3584):
        w = synth.q4k_matrix(out_dim, in_dim, rng)
        wd, yd = upload(w), DeviceBuffer(out_dim * 4)
        assert cuda.mg_matvec_q4k_limbs_on_stream(wd.ptr, rec.ptr, None, yd.ptr, out_dim, in_dim // 256, None) == 0
        kern.sync()
        assert rel_rms_err(yd.copy_to_host(out_dim), orc.matvec_f64(w, x, out_dim, in_dim // 256)) <= GEMV_TOL
    # the records reproduce x to 2^-22 of each sub-block's maximum
    words = np.empty(nbytes // 4, dtype=np.uint32)
    assert cuda.mg_memcpy_d2h(words.ctypes.data_as(C.c_void_p), rec.ptr, nbytes) == 0
    r = words.reshape(-1, 52)
    planes = r[:, :48].reshape(-1, 2, 3, 8).view(np.uint8).reshape(-1, 2, 3, 32)
    a = (planes[:, :, 0].view(np.int8).astype(np.int64) * 65536 + planes[:, :, 1].astype(np.int64) * 256
         + planes[:, :, 2].astype(np.int64))
    s = r[:, 48:50].copy().view(np.float32)
    xr = (a * s[:, :, None].astype(np.float64)).reshape(-1)
    xs = x.reshape(-1, 32)
    bound = np.repeat(np.abs(xs).max(1) * 2.0 ** -22, 32)
    assert np.all(np.abs(xr - x) <= bound)
    assert np.allclose(r[:, 50:52].copy().view(np.float32).reshape(-1), xr.reshape(-1, 32).sum(1), rtol=1e-6, atol=1e-6)
    assert cuda.mg_q4k_x_to_limbs_on_stream(xd.ptr, 100, rec.ptr, None) == 1


def test_matvec_heavy_tailed_and_nonfinite_activations(orc):
    out_dim, bpr = 64, 6
    rng = np.random.Generator(np.random.PCG64(99))
    w = synth.q4k_matrix(out_dim, bpr * 256, rng)
    x = synth.activations(bpr * 256, rng)
    heavy = (x * np.exp(3.0 * rng.standard_normal(x.shape))).astype(np.float32)
    assert rel_rms_err(gpu_matvec(w, heavy, out_dim, bpr), orc.matvec_f64(w, heavy, out_dim, bpr)) <= GEMV_TOL
    tiny = (x * np.float32(1e-30)).astype(np.float32)
    assert rel_rms_err(gpu_matvec(w, tiny, out_dim, bpr), orc.matvec_f64(w, tiny, out_dim, bpr)) <= GEMV_TOL
    zero = np.zeros_like(x)
    assert np.array_equal(gpu_matvec(w, zero, out_dim, bpr), np.zeros(out_dim, np.float32))
    # NaN in x reaches every row, as w * NaN does in the reference's accumulation
    bad = x.copy()
    bad[300] = np.nan
    assert np.all(np.isnan(gpu_matvec(w, bad, out_dim, bpr)))


def test_matvec_very_long_rows_take_the_f32_variant(orc):
    check_matvec(orc, 24, 250, 4242)


def test_zz_no_gemv_wait_ever_ran_out(cuda):
    """Every wait inside the GEMV kernels is bounded; none of the launches above may have given up."""
    assert cuda.mg_matvec_q4k_timeouts() == 0

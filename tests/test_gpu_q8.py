"""GPU parity of the int8-activation pair (launch_quantize_q8_1 / launch_matvec_q4k_dp4a) through
the C ABI, against the oracle's restatement of crates/modgrad-device/kernels/matvec_q4k_dp4a.hip.

Quantised activations: bit-exact (int8 values, f32 scales and sums).  Matvec on the SAME int8
inputs: 1e-5 of the output RMS.  Against the f32 path: RMS-relative below 2 %, the reference's own
acceptance bound for this lossy path (examples/rocm_dp4a_check.rs:63-65)."""
import numpy as np
import pytest

from conftest import GEMV_TOL, rel_rms_err, rms
from modgrad_b200 import synth
from modgrad_b200.backend import DeviceBuffer, kern

pytestmark = pytest.mark.gpu


def upload(a: np.ndarray) -> DeviceBuffer:
    a = np.ascontiguousarray(a)
    b = DeviceBuffer(a.nbytes)
    b.copy_from_host_bytes(a)
    return b


def gpu_quantize(x):
    n = x.size
    xd_, xq, xd, xs = upload(x), DeviceBuffer(n), DeviceBuffer(n // 32 * 4), DeviceBuffer(n // 32 * 4)
    kern.quantize_q8_1(xd_.ptr, xq.ptr, xd.ptr, xs.ptr, n)
    kern.sync()
    q = np.empty(n // 32 * 32, dtype=np.int8)
    xq.copy_to_host_bytes(q.view(np.uint8))
    return q, xd.copy_to_host(n // 32), xs.copy_to_host(n // 32), (xq, xd, xs)


@pytest.mark.parametrize("n", [32, 256, 3584, 18944, 8192 + 17])
def test_quantize_q8_1_bit_exact(orc, n):
    rng = np.random.Generator(np.random.PCG64(500 + n))
    x = synth.activations(n, rng)
    x[: min(n, 32)] = 0.0                      # an all-zero sub-block: scale 0, zeros
    if n >= 96:
        x[32:64] *= np.float32(1e-42)          # denormal amax: 127/amax overflows -> zero sub-block
        x[64] = 1e30
    q, xd, xs, _ = gpu_quantize(x)
    oq, od, osum = orc.quantize_q8_1(x)
    m = n // 32 * 32
    assert np.array_equal(q, oq[:m])
    assert np.array_equal(xd.view(np.uint32), od.view(np.uint32))
    assert np.array_equal(xs.view(np.uint32), osum.view(np.uint32))


@pytest.mark.parametrize("out_dim,bpr", [(4096, 16), (512, 14), (3584, 74), (18944, 14), (33, 5), (1, 1), (7, 113)])
def test_matvec_q4k_dp4a_matches_reference_arithmetic(orc, out_dim, bpr):
    rng = np.random.Generator(np.random.PCG64(900 + out_dim + bpr))
    w = synth.q4k_matrix(out_dim, bpr * 256, rng)
    x = synth.activations(bpr * 256, rng)
    q, xd, xs, (dq, dd, ds) = gpu_quantize(x)
    wd, yd = upload(w), DeviceBuffer(out_dim * 4)
    kern.matvec_q4k_dp4a(wd.ptr, dq.ptr, dd.ptr, ds.ptr, yd.ptr, out_dim, bpr)
    kern.sync()
    y = yd.copy_to_host(out_dim)
    want = orc.matvec_q8_1(w, q, xd, xs, out_dim, bpr).astype(np.float64)
    assert rel_rms_err(y, want) <= GEMV_TOL
    # the lossy path against the f32 one (the reference's acceptance bound: RMS-relative < 2 %)
    y64 = orc.matvec_f64(w, x, out_dim, bpr)
    if out_dim >= 32:
        assert rms(y - y64) / rms(y64) < 0.02


def test_matvec_q4k_dp4a_nonfinite_sum_is_zero_and_bad_arguments(orc, cuda):
    out_dim, bpr = 16, 2
    rng = np.random.Generator(np.random.PCG64(31))
    w = synth.q4k_matrix(out_dim, bpr * 256, rng)
    x = synth.activations(bpr * 256, rng)
    q, xd, xs, (dq, dd, ds) = gpu_quantize(x)
    bad = xd.copy()
    bad[3] = np.inf                              # a degenerate scale: every row sum becomes non-finite
    dd.copy_from_host(bad)
    wd, yd = upload(w), DeviceBuffer(out_dim * 4)
    kern.matvec_q4k_dp4a(wd.ptr, dq.ptr, dd.ptr, ds.ptr, yd.ptr, out_dim, bpr)
    kern.sync()
    assert np.array_equal(yd.copy_to_host(out_dim), np.zeros(out_dim, np.float32))   # matvec_q4k_dp4a.hip:104-106
    assert cuda.launch_matvec_q4k_dp4a(wd.ptr, dq.ptr, dd.ptr, ds.ptr, yd.ptr, 0, bpr) == 1   # hipErrorInvalidValue
    assert cuda.launch_matvec_q4k_dp4a(wd.ptr, dq.ptr, dd.ptr, ds.ptr, yd.ptr, out_dim, 0) == 1
    assert cuda.launch_quantize_q8_1(None, dq.ptr, dd.ptr, ds.ptr, 64) == 1

"""GPU parity of the tensor-core (tcgen05) multi-sequence Q4_K dequant-GEMM against M
independent matvecs of the CPU oracle on the SAME f32 activations (the batched contract of
Linear::forward_batched, crates/modgrad-device/src/backend/tensor.rs:1839-1853).  The kernel
carries each activation as two half-precision limbs (22 significant bits relative to the
sequence's largest magnitude), which keeps it inside the 1e-5 bound of the batch-1 path."""
import ctypes as C

import numpy as np
import pytest

from conftest import GEMV_TOL, rms
from modgrad_b200 import synth
from modgrad_b200.backend import DeviceBuffer, kern

pytestmark = pytest.mark.gpu

CANARY = 4096  # floats behind Y that the kernel must leave alone


def up(a):
    a = np.ascontiguousarray(a)
    b = DeviceBuffer(a.nbytes)
    b.copy_from_host_bytes(a)
    return b


def aligned_scratch(nbytes):
    buf = DeviceBuffer(nbytes + 1024)
    return buf, (buf.ptr + 1023) & ~1023


def gpu_matmul(cuda, w, x, m, out_dim, bpr):
    """Y holds exactly m * out_dim floats; a canary region follows and is checked."""
    wd, xd, yd = up(w), up(x), DeviceBuffer((m * out_dim + CANARY) * 4)
    yd.copy_from_host(np.full(m * out_dim + CANARY, -777.0, dtype=np.float32))
    nbytes = cuda.mg_matmul_q4k_scratch_bytes(m, bpr)
    keep, scratch = aligned_scratch(nbytes)
    assert cuda.launch_matmul_q4k_on_stream(wd.ptr, xd.ptr, yd.ptr, m, out_dim, bpr, scratch, None) == 0
    kern.sync()
    assert cuda.mg_matmul_q4k_status(scratch, m, bpr) == 0, "a bounded wait inside the kernel expired"
    out = yd.copy_to_host(m * out_dim + CANARY)
    assert np.all(out[m * out_dim:] == -777.0), "the kernel wrote past m_rows * out_dim"
    return out[:m * out_dim].reshape(m, out_dim)


def check(cuda, orc, m, out_dim, bpr, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    w = synth.q4k_matrix(out_dim, bpr * 256, rng)
    x = synth.activations(bpr * 256, rng, rows=m)
    y = gpu_matmul(cuda, w, x, m, out_dim, bpr)
    worst = 0.0
    for i in range(m):
        ref = orc.matvec_f64(w, x[i], out_dim, bpr)
        worst = max(worst, float(np.max(np.abs(y[i] - ref)) / rms(ref)))
    assert worst <= GEMV_TOL, f"M={m} {out_dim}x{bpr * 256}: {worst:.3e}"
    return worst


def test_matmul_tc_smallest_tile(cuda, orc):
    check(cuda, orc, 16, 128, 1, 1)


@pytest.mark.parametrize("m,out_dim,bpr", [(16, 256, 2), (5, 130, 3), (1, 128, 1), (32, 384, 4), (64, 512, 5), (33, 1000, 7),
                                           (64, 128, 40), (17, 19000, 2), (48, 100, 9)])
def test_matmul_tc_shapes(cuda, orc, m, out_dim, bpr):
    check(cuda, orc, m, out_dim, bpr, 100 + m + out_dim + bpr)


@pytest.mark.parametrize("m", [16, 32, 64])
@pytest.mark.parametrize("shape", [(18944, 3584), (3584, 18944)])
def test_matmul_tc_7b_shapes_sampled_rows(cuda, orc, m, shape):
    """Full-size operands; the oracle checks a sample of output rows (all M sequences)."""
    out_dim, in_dim = shape
    bpr = in_dim // 256
    rng = np.random.Generator(np.random.PCG64(m + out_dim))
    w = synth.q4k_matrix(out_dim, in_dim, rng)
    x = synth.activations(in_dim, rng, rows=m)
    y = gpu_matmul(cuda, w, x, m, out_dim, bpr)
    rows = np.unique(np.concatenate([np.arange(0, 256), rng.integers(0, out_dim, 512), np.arange(out_dim - 130, out_dim)]))
    wr = w.reshape(out_dim, -1)[rows].reshape(-1)
    for i in range(0, m, max(1, m // 8)):
        ref = orc.matvec_f64(wr, x[i], rows.size, bpr)
        assert float(np.max(np.abs(y[i][rows] - ref)) / rms(ref)) <= GEMV_TOL
    # and every sequence equals the batch-1 kernel on the same activations
    xd, yd, wd = up(x[m - 1]), DeviceBuffer(out_dim * 4), up(w)
    kern.matvec_q4k(wd.ptr, xd.ptr, yd.ptr, out_dim, bpr)
    kern.sync()
    y1 = yd.copy_to_host(out_dim)
    assert float(np.max(np.abs(y[m - 1] - y1)) / rms(y1)) <= 2 * GEMV_TOL


def test_matmul_tc_rejects_bad_arguments(cuda):
    buf = DeviceBuffer(4096)
    p = (buf.ptr + 1023) & ~1023
    assert cuda.launch_matmul_q4k_on_stream(p, p, p, 0, 128, 1, p, None) == 1
    assert cuda.launch_matmul_q4k_on_stream(p, p, p, 65, 128, 1, p, None) == 1
    assert cuda.launch_matmul_q4k_on_stream(p, p, p, 16, 128, 1, p + 16, None) == 1
    assert cuda.launch_matmul_q4k_on_stream(p, p, p, 16, 128, 1, None, None) == 1

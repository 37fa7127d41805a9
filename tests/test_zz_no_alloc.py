"""The allocation-free matvec entry point, for hosts that manage every byte of device memory
themselves (an arena-based engine, a fixed-budget server) and so cannot let a library call
cudaMalloc on their behalf.  It must give what the ordinary entry point gives, also on a second
call in a row (the built-in scratch array keeps the previous call's contents), for short rows,
for rows long enough that the ordinary path uses run-time scratch, and it must refuse rows
beyond its fixed capacity."""
import numpy as np
import pytest

from conftest import GEMV_TOL, rel_rms_err
from modgrad_b200 import synth
from modgrad_b200.backend import DeviceBuffer, kern

pytestmark = pytest.mark.gpu


def up(a):
    a = np.ascontiguousarray(a)
    b = DeviceBuffer(a.nbytes)
    b.copy_from_host_bytes(a)
    return b


def test_noalloc_matvec_matches_ordinary_entry_point_twice_in_a_row(cuda):
    for out_dim, bpr in [(3584, 74), (512, 14)]:          # long rows (scratch path) and short rows
        rng = np.random.Generator(np.random.PCG64(out_dim + bpr))
        w = synth.q4k_matrix(out_dim, bpr * 256, rng)
        wd = up(w)
        for call in range(2):                              # two calls in a row, different activations
            x = synth.activations(bpr * 256, rng)
            xd, y_ref, y_new = up(x), DeviceBuffer(out_dim * 4), DeviceBuffer(out_dim * 4)
            assert cuda.launch_matvec_q4k_on_stream(wd.ptr, xd.ptr, y_ref.ptr, out_dim, bpr, None) == 0
            assert cuda.launch_matvec_q4k_noalloc_on_stream(wd.ptr, xd.ptr, y_new.ptr, out_dim, bpr, None) == 0
            kern.sync()
            a, b = y_ref.copy_to_host(out_dim), y_new.copy_to_host(out_dim)
            assert np.all(np.isfinite(b))
            assert rel_rms_err(b, a.astype(np.float64)) <= GEMV_TOL, (out_dim, bpr, call)


def test_noalloc_calls_queued_back_to_back_share_the_array_safely(cuda):
    """Three calls queued on one stream with no synchronisation in between, each with its own x and y:
    every kernel waits for its predecessor to complete before it rewrites the shared array, so each
    result must equal the ordinary entry point's."""
    out_dim, bpr = 2048, 40
    rng = np.random.Generator(np.random.PCG64(17))
    wd = up(synth.q4k_matrix(out_dim, bpr * 256, rng))
    xs = [up(synth.activations(bpr * 256, rng)) for _ in range(3)]
    ys = [DeviceBuffer(out_dim * 4) for _ in range(3)]
    refs = [DeviceBuffer(out_dim * 4) for _ in range(3)]
    for x, y in zip(xs, ys):
        assert cuda.launch_matvec_q4k_noalloc_on_stream(wd.ptr, x.ptr, y.ptr, out_dim, bpr, None) == 0
    for x, r in zip(xs, refs):
        assert cuda.launch_matvec_q4k_on_stream(wd.ptr, x.ptr, r.ptr, out_dim, bpr, None) == 0
    kern.sync()
    for y, r in zip(ys, refs):
        assert rel_rms_err(y.copy_to_host(out_dim), r.copy_to_host(out_dim).astype(np.float64)) <= GEMV_TOL
    assert cuda.mg_matvec_q4k_timeouts() == 0


def test_noalloc_matvec_refuses_rows_beyond_its_capacity(cuda):
    buf = DeviceBuffer(4096)
    assert cuda.launch_matvec_q4k_noalloc_on_stream(buf.ptr, buf.ptr, buf.ptr, 4, 129, None) == 1
    assert cuda.launch_matvec_q4k_noalloc_on_stream(buf.ptr, buf.ptr, buf.ptr, 0, 4, None) == 1

"""Q4_K residency container (LinearResidentQuantized, crates/modgrad-compute/src/neuron.rs:866-1250) and
its host quantiser.  The reference's own tests are mirrored: quantised forward vs fp32 forward
RMS-relative < 10 % (neuron.rs:1885-1941), evict -> re-dequantise bit-identical (:1943-1994), host size
below 16 % of fp32 (:1996-2024), quantise -> dequantise round trip below 5 % RMS on a smooth signal
(crates/modgrad-device/src/kfd/gguf.rs:703-738)."""
import numpy as np
import pytest

from conftest import GEMV_TOL, rel_rms_err, rms
from modgrad_b200 import residency
from modgrad_b200.backend import DeviceBuffer, Runtime, kern


def smooth_signal(n):
    i = np.arange(n, dtype=np.float32)
    return (np.sin(i * np.float32(0.01)) * np.float32(0.5) + np.cos(i * np.float32(0.003)) * np.float32(0.3)).astype(np.float32)


def test_quantize_round_trip_within_five_percent(orc):
    # the reference's smooth signal: below 5 %; white Gaussian noise (sixteen levels across +-2 sigma): below 10 %
    for x, bound in ((smooth_signal(256 * 16), 0.05),
                     (np.random.Generator(np.random.PCG64(3)).standard_normal(256 * 64).astype(np.float32), 0.10)):
        q = residency.quantize_row_q4_k(x)
        assert q.size == x.size // 256 * 144
        back = orc.dequantize(q)                      # the canonical-order dequantiser of the reference
        assert rms(back - x) / rms(x) < bound
    z = np.zeros(512, np.float32)
    assert np.array_equal(orc.dequantize(residency.quantize_row_q4_k(z)), z)
    with pytest.raises(Runtime):
        residency.quantize_row_q4_k(np.zeros(100, np.float32))


def test_dequant_is_a_pure_function_of_the_quantised_bytes(orc):
    x = smooth_signal(256 * 4)
    a, b = residency.quantize_row_q4_k(x), residency.quantize_row_q4_k(x.copy())
    assert np.array_equal(a, b) and np.array_equal(orc.dequantize(a).view(np.uint32), orc.dequantize(b).view(np.uint32))


def test_host_size_savings():
    w = np.random.Generator(np.random.PCG64(4)).standard_normal((1024, 1024)).astype(np.float32)
    lin = residency.LinearResidentQuantized.from_linear(w, np.zeros(1024, np.float32))
    assert not lin.is_resident()                                   # from_linear allocates nothing on the device
    ratio = lin.host_size_bytes() / (w.size * 4)
    assert lin.host_size_bytes() < w.size and ratio < 0.16
    lin.close()
    with pytest.raises(Runtime):
        residency.LinearResidentQuantized.from_linear(np.zeros((4, 100), np.float32))


def up(a):
    b = DeviceBuffer(a.nbytes)
    b.copy_from_host_bytes(a)
    return b


@pytest.mark.gpu
@pytest.mark.parametrize("expanded", [False, True])
def test_quantized_forward_close_to_fp32_forward(orc, expanded):
    in_dim, out_dim = 1024, 256
    rng = np.random.Generator(np.random.PCG64(0xCAFE))
    w = (rng.standard_normal((out_dim, in_dim)) / np.sqrt(in_dim)).astype(np.float32)
    bias = rng.standard_normal(out_dim).astype(np.float32)
    x = rng.standard_normal(in_dim).astype(np.float32)
    ref = w.astype(np.float64) @ x.astype(np.float64) + bias
    lin = residency.LinearResidentQuantized.from_linear(w, bias)
    lin.set_expanded(expanded)
    xd, yd = up(x), DeviceBuffer(out_dim * 4)
    lin.forward(xd, yd, auto_evict=False)
    kern.sync()
    y = yd.copy_to_host(out_dim)
    assert lin.is_resident()
    assert rms(y - ref) / rms(ref) < 0.10
    # and exact (to the matvec tolerance) against the oracle on the quantised bytes themselves
    want = orc.matvec_f64(lin.host_blocks(), x, out_dim, in_dim // 256) + bias
    assert rel_rms_err(y, want) <= GEMV_TOL
    assert lin.device_size_bytes() == lin.host_size_bytes() + (in_dim * out_dim * 4 if expanded else 0)
    lin.close()


@pytest.mark.gpu
@pytest.mark.parametrize("expanded", [False, True])
def test_evict_then_forward_is_bit_identical(expanded):
    in_dim, out_dim = 512, 128
    rng = np.random.Generator(np.random.PCG64(0xC0FFEE))
    lin = residency.LinearResidentQuantized.from_linear(rng.standard_normal((out_dim, in_dim)).astype(np.float32))
    lin.set_expanded(expanded)
    xd = up(rng.standard_normal(in_dim).astype(np.float32))
    ya, yb = DeviceBuffer(out_dim * 4), DeviceBuffer(out_dim * 4)
    lin.forward(xd, ya, auto_evict=True)
    assert not lin.is_resident()                      # auto_evict drops the device buffers after the dispatch
    lin.forward(xd, yb, auto_evict=False)
    kern.sync()
    assert lin.is_resident()
    assert np.array_equal(ya.copy_to_host(out_dim).view(np.uint32), yb.copy_to_host(out_dim).view(np.uint32))
    lin.evict()
    assert not lin.is_resident()
    lin.close()


@pytest.mark.gpu
def test_direct_and_expanded_modes_agree(orc):
    in_dim, out_dim = 3584, 512
    rng = np.random.Generator(np.random.PCG64(5))
    from modgrad_b200 import synth
    blocks = synth.q4k_matrix(out_dim, in_dim, rng)
    x = synth.activations(in_dim, rng)
    lin = residency.LinearResidentQuantized.from_blocks(blocks, in_dim, out_dim)
    xd, y1, y2 = up(x), DeviceBuffer(out_dim * 4), DeviceBuffer(out_dim * 4)
    lin.forward(xd, y1)
    lin.set_expanded(True)
    lin.forward(xd, y2)
    kern.sync()
    want = orc.matvec_f64(blocks, x, out_dim, in_dim // 256)
    assert rel_rms_err(y1.copy_to_host(out_dim), want) <= GEMV_TOL
    assert rel_rms_err(y2.copy_to_host(out_dim), want) <= GEMV_TOL
    lin.close()

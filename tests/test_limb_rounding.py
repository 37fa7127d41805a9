"""The integer matvec kernels (Q4_K, Q5_K, Q6_K) multiply exact quants with activations rounded to a
block-fixed-point form: per 32-element sub-block one power-of-two scale s = 2^(floor(log2 max|x|) - 21)
and integers a = rint(x / s), |a| <= 2^22 (modgrad_b200/csrc/xlimbs.cuh).  Everything after that rounding is
exact integer arithmetic, so the distance of those kernels from the f64 dot product is the distance this
restatement measures on the CPU: far inside the 1e-5 contract of the GPU tests."""
import numpy as np

from modgrad_b200 import synth
from oracle import q4k_numpy as qn


def limb_round(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32).reshape(-1, 32)
    amax = np.max(np.abs(x), axis=1, keepdims=True).astype(np.float64)
    e = np.where(amax > 0, np.floor(np.log2(np.where(amax > 0, amax, 1.0))), -127.0)
    e = np.maximum(e, -100.0)
    s = np.exp2(e - 21.0)
    a = np.rint(x.astype(np.float64) / s)
    assert np.max(np.abs(a)) <= 2 ** 22
    return (a * s).reshape(-1)


def test_rounded_activations_stay_inside_the_contract():
    rng = np.random.Generator(np.random.PCG64(123))
    for kind, rows, bpr in ((6, 64, 14), (5, 64, 14), (6, 16, 74)):
        w = synth.kquant_matrix(kind, rows, bpr * 256, rng)
        dq = (qn.dequantize_q6k if kind == 6 else qn.dequantize_q5k)(w.reshape(-1, 210 if kind == 6 else 176))
        dq = dq.reshape(rows, bpr * 256).astype(np.float64)
        # activations with a wide spread inside each sub-block: the worst case for a shared scale
        x = (rng.standard_normal(bpr * 256) * np.exp(rng.uniform(-6, 6, bpr * 256))).astype(np.float32)
        exact = dq @ x.astype(np.float64)
        rounded = dq @ limb_round(x)
        err = np.max(np.abs(rounded - exact)) / np.sqrt(np.mean(exact ** 2))
        assert err < 2e-6, (kind, rows, bpr, err)
    # a sub-block of zeros and one of sub-normals survive the scale computation
    z = np.zeros(64, dtype=np.float32)
    z[32:] = 1e-41
    assert np.all(np.isfinite(limb_round(z)))

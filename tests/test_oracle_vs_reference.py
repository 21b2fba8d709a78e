"""The plain-C oracle against the reference itself (compiled from its sources into oracle/_ref) on fresh
random inputs.  Skipped where the compiled reference is absent."""
import numpy as np
import pytest

import inputs
from oracle.binding import Q4_0, Q8_0, Q8_AVX2, Q8_SCALAR


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_quantisers_bit_exact(oracle, reference, seed):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((64, 4096)) * rng.choice([1e-3, 1.0, 50.0], (64, 1))).astype(np.float32)
    for v in (Q8_AVX2, Q8_SCALAR):
        assert np.array_equal(oracle.quantize_q8_0(x, v), reference.quantize_q8_0(x, v))
    w = (rng.standard_normal((32, 2048)) * 0.02).astype(np.float32)
    for t in (Q4_0, Q8_0):
        assert np.array_equal(oracle.quantize_weights(t, w), reference.quantize_weights(t, w))


@pytest.mark.parametrize("wtype", [Q4_0, Q8_0])
@pytest.mark.parametrize("shape", [(33, 64, 1), (128, 4096, 9), (17, 14336, 2)])
def test_mul_mat_bit_exact(oracle, reference, wtype, shape):
    M, K, N = shape
    rng = np.random.default_rng(M * 7 + N)
    wq = reference.quantize_weights(wtype, (rng.standard_normal((M, K)) * 0.02).astype(np.float32))
    x = rng.standard_normal((N, K)).astype(np.float32)
    a, _ = oracle.mul_mat(wtype, wq, x)
    b, _ = reference.mul_mat(wtype, wq, x, n_threads=3)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_flash_attn_bit_exact(oracle, reference):
    c = inputs.ragged_case(900, 128, 8, 2, 512, [(120, 2), (255, 1), (60, 4)])
    a = oracle.flash_attn_ext(c["q"], c["kc"], c["vc"], c["mask"], c["scale"], n_kv=c["n_kv"])
    b, _ = reference.flash_attn_ext(c["q"], c["kc"], c["vc"], c["mask"], c["scale"], n_kv=c["n_kv"], n_threads=2)
    v = c["valid_rows"]
    assert np.array_equal(a[v].view(np.uint32), b[v].view(np.uint32))

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


@pytest.mark.parametrize("D,H,Hkv,max_bias,softcap", [(64, 8, 8, 0.0, 0.0),      # head size 64 (the 1B architecture), no grouping
                                                     (128, 12, 4, 8.0, 0.0),    # ALiBi slopes, a head count that is no power of two
                                                     (128, 8, 2, 0.0, 30.0),    # logit soft-capping
                                                     (64, 6, 2, 4.0, 50.0)])    # both
def test_flash_attn_bias_and_softcap_bit_exact(oracle, reference, D, H, Hkv, max_bias, softcap):
    """The branches of the reference's attention a llama graph does not take (cactus/ggml-cpu/ops.cpp:6990-7010 slopes,
    :7093-7096 soft-capping) follow the same arithmetic in the restatement."""
    c = inputs.ragged_case(D + H, D, H, Hkv, 512, [(77, 3), (130, 1), (256, 5)])
    a = oracle.flash_attn_ext(c["q"], c["kc"], c["vc"], c["mask"], c["scale"], max_bias=max_bias, softcap=softcap, n_kv=c["n_kv"])
    b, _ = reference.flash_attn_ext(c["q"], c["kc"], c["vc"], c["mask"], c["scale"], max_bias=max_bias, softcap=softcap, n_kv=c["n_kv"], n_threads=2)
    v = c["valid_rows"]
    assert np.array_equal(a[v].view(np.uint32), b[v].view(np.uint32))


def test_quantisers_on_zero_rows_ties_and_tiny_values(oracle, reference):
    """Edge values of the quantisers: all-zero blocks (scale 0, inverse 0), values on rounding ties, blocks whose scale is a
    subnormal half, one outlier per block."""
    rng = np.random.default_rng(11)
    x = np.zeros((8, 256), np.float32)
    x[1] = (rng.integers(-254, 255, 256) * 0.5).astype(np.float32)        # with the block maximum 127 every value is a tie or exact
    x[1, ::32] = 127.0
    x[2] = (rng.standard_normal(256) * 1e-7).astype(np.float32)           # d = max / 127 below the smallest normal half
    x[3] = rng.standard_normal(256).astype(np.float32)
    x[3, 5::32] = 1000.0                                                  # one outlier per block
    x[4, :32] = -1.0                                                      # a constant block next to zero blocks
    x[5] = np.float32(65504.0) * rng.choice([-1.0, 1.0], 256).astype(np.float32)
    x[6] = rng.standard_normal(256).astype(np.float32) * np.float32(2.0) ** rng.integers(-20, 10, 256).astype(np.float32)
    for v in (Q8_AVX2, Q8_SCALAR):
        assert np.array_equal(oracle.quantize_q8_0(x, v), reference.quantize_q8_0(x, v)), v
    for t in (Q4_0, Q8_0):
        assert np.array_equal(oracle.quantize_weights(t, x), reference.quantize_weights(t, x)), t


@pytest.mark.parametrize("wtype", [Q4_0, Q8_0])
def test_mul_mat_one_block_rows_and_zero_weights(oracle, reference, wtype):
    """The smallest row (one 32-element block), a weight row of zeros (block scale 0) and a zero activation row."""
    rng = np.random.default_rng(13)
    for M, K, N in ((1, 32, 1), (5, 32, 3), (16, 96, 4)):
        w = (rng.standard_normal((M, K)) * 0.05).astype(np.float32)
        w[0] = 0.0
        wq = reference.quantize_weights(wtype, w)
        x = rng.standard_normal((N, K)).astype(np.float32)
        x[-1] = 0.0
        a, _ = oracle.mul_mat(wtype, wq, x)
        b, _ = reference.mul_mat(wtype, wq, x, n_threads=2)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), (M, K, N)
        assert (a[-1] == 0).all() and (a[:, 0] == 0).all()

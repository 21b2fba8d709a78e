"""K1 on the GPU: quantize_row_q8_0 must be byte-identical to the reference (both arithmetic variants),
and the tiled weight layout must round-trip exactly."""
import numpy as np
import pytest
import torch

import inputs
from gpu_util import dev, host
from oracle.binding import Q4_0, Q8_0, Q8_AVX2, Q8_SCALAR

pytestmark = pytest.mark.gpu


def test_q8_0_matches_golden_both_variants(golden):
    from cactus_b200 import ops
    x = dev(inputs.quantizer_rows())
    assert np.array_equal(host(ops.quantize_row_q8_0(x, Q8_AVX2)), golden["q8_avx2"])
    assert np.array_equal(host(ops.quantize_row_q8_0(x, Q8_SCALAR)), golden["q8_scalar"])


@pytest.mark.parametrize("shape", [(1, 32), (3, 4096), (64, 14336), (513, 2048)])
def test_q8_0_matches_oracle_random(oracle, shape):
    from cactus_b200 import ops
    rng = np.random.default_rng(shape[0] + shape[1])
    x = (rng.standard_normal(shape) * rng.choice([1e-4, 1.0, 300.0], (shape[0], 1))).astype(np.float32)
    for v in (Q8_AVX2, Q8_SCALAR):
        assert np.array_equal(host(ops.quantize_row_q8_0(dev(x), v)), oracle.quantize_q8_0(x, v))


def test_q8_0_strided_rows(oracle):
    from cactus_b200 import ops
    rng = np.random.default_rng(5)
    big = rng.standard_normal((9, 1000)).astype(np.float32)
    xd = dev(big)[:, 8:8 + 256]          # row stride 1000 floats, 32-byte offset
    assert np.array_equal(host(ops.quantize_row_q8_0(xd)), oracle.quantize_q8_0(big[:, 8:264]))
    xd = dev(big)[:, 3:3 + 256]          # rows not 16-byte aligned: scalar load path
    assert np.array_equal(host(ops.quantize_row_q8_0(xd)), oracle.quantize_q8_0(big[:, 3:259]))


def test_q8_0_full_size_idempotence_property():
    """At config-1 size (512 x 4096): quantising the dequantised blocks reproduces the same blocks."""
    from cactus_b200 import ops
    x = dev(inputs.cfg1_activations(512))
    q = ops.quantize_row_q8_0(x)
    blocks = q.view(512, 128, 34)
    d = blocks[:, :, :2].contiguous().view(torch.float16).float()          # [512,128,1]
    qs = blocks[:, :, 2:].contiguous().view(torch.int8).float()            # [512,128,32]
    x2 = (qs * d).reshape(512, 4096).contiguous()
    q2 = ops.quantize_row_q8_0(x2)
    # quants are reproduced exactly; the scale may move by one fp16 ulp (d is rounded to fp16 twice)
    assert torch.equal(q2.view(512, 128, 34)[:, :, 2:], blocks[:, :, 2:])


@pytest.mark.parametrize("wtype", [Q4_0, Q8_0])
@pytest.mark.parametrize("shape", [(16, 128), (33, 64), (24, 256), (100, 96), (4096, 4096)])
def test_tiled_weight_layout_round_trip(oracle, wtype, shape):
    from cactus_b200 import ops
    M, K = shape
    rng = np.random.default_rng(M + K)
    bb = 18 if wtype == Q4_0 else 34
    blocks = rng.integers(0, 256, (M, K // 32 * bb), dtype=np.uint8)   # any byte pattern must survive
    w = ops.QWeight.from_blocks(wtype, K, M, blocks)
    assert np.array_equal(host(w.to_blocks()), blocks)


def test_tiled_weight_partial_upload(oracle):
    """A loader may upload a tensor in row ranges; the result equals a single upload."""
    from cactus_b200 import ops
    from cactus_b200._lib import check, lib
    M, K = 100, 256
    rng = np.random.default_rng(77)
    blocks = rng.integers(0, 256, (M, K // 32 * 18), dtype=np.uint8)
    whole = ops.QWeight.from_blocks(Q4_0, K, M, blocks)
    L = lib()
    data = torch.zeros_like(whole.data)
    src = dev(blocks)
    row_bytes = K // 32 * 18
    for r0, cnt in ((0, 32), (32, 48), (80, 20)):
        check(L.b200_weight_upload(Q4_0, K, M, src.data_ptr() + r0 * row_bytes, data.data_ptr(), r0, cnt, None))
    torch.cuda.synchronize()
    assert torch.equal(data, whole.data)
    # bad ranges are refused
    assert L.b200_weight_upload(Q4_0, K, M, src.data_ptr(), data.data_ptr(), 8, 16, None) == -1
    assert L.b200_weight_upload(Q4_0, K, M, src.data_ptr(), data.data_ptr(), 0, 200, None) == -1


def test_get_rows_on_tiled_table(oracle):
    from cactus_b200 import ops
    rng = np.random.default_rng(11)
    for wtype in (Q4_0, Q8_0):
        w = (rng.standard_normal((70, 128)) * 0.02).astype(np.float32)
        wq = oracle.quantize_weights(wtype, w)
        ids = np.array([0, 69, 3, 3, 17, 9, 15, 30, 60, 8], np.int32)   # rows in both halves of a 16-row tile
        got = host(ops.get_rows(ops.QWeight.from_blocks(wtype, 128, 70, wq), dev(ids)))
        assert np.array_equal(got.view(np.uint32), oracle.get_rows(wtype, wq, ids, 128).view(np.uint32))

"""K6 on the GPU: the small row ops of a llama layer against the golden vectors of the reference."""
import numpy as np
import pytest
import torch

import inputs
from gpu_util import dev, host

pytestmark = pytest.mark.gpu


def test_row_ops_vs_golden(golden):
    from cactus_b200 import ops
    r = inputs.row_op_inputs()
    x, y, w = dev(r["x"]), dev(r["y"]), dev(r["w"])
    np.testing.assert_allclose(host(ops.rms_norm(x, 1e-5, w)), golden["rms"], rtol=0, atol=2e-6)
    assert np.array_equal(host(ops.add(x, y)).view(np.uint32), golden["add"].view(np.uint32))
    np.testing.assert_allclose(host(ops.silu(x, y)), golden["silu_mul"], rtol=0, atol=1e-5)
    np.testing.assert_allclose(host(ops.rope_ext(dev(r["xr"]), dev(r["pos"]), 128, 500000.0)), golden["rope"], rtol=0, atol=2e-5)
    dst = torch.zeros((7, 2048), dtype=torch.float16, device="cuda")
    ops.cpy(x, dst)
    assert np.array_equal(host(dst).view(np.uint16), golden["cpy_f16"])


def test_mul_broadcast_and_views(oracle):
    from cactus_b200 import ops
    rng = np.random.default_rng(1)
    a = rng.standard_normal((5, 64)).astype(np.float32)
    w = rng.standard_normal(64).astype(np.float32)
    assert np.array_equal(host(ops.mul(dev(a), dev(w))), a * w)
    # CPY into a strided slice of a larger f16 buffer (a KV-cache view)
    cache = torch.zeros((16, 64), dtype=torch.float16, device="cuda")
    ops.cpy(dev(a), cache[4:9])
    got = host(cache)
    assert np.array_equal(got[4:9].view(np.uint16), oracle.cpy_f32_f16(a))
    assert (got[:4] == 0).all() and (got[9:] == 0).all()
    # GET_ROWS on an f32 table
    ids = np.array([4, 0, 4], np.int32)
    assert np.array_equal(host(ops.get_rows(dev(a), dev(ids))), a[ids])


def test_k_shift_rope_f16_and_f16_copy(golden):
    """K-shift (ROPE in place on cached f16 keys) against the reference's golden vector, and the f16 row copies a cache
    defragmentation issues.  sinf/cosf of the device differ from glibc's in the last bit, so a result may land one f16
    step away; rows with a zero shift must come back bit for bit."""
    from cactus_b200._lib import check, lib
    L = lib()
    r = inputs.row_op_inputs()
    k = torch.from_numpy(r["kf16"].view(np.int16)).cuda()          # [cells, kv heads, D] f16 bits
    shift = torch.from_numpy(r["shift"]).cuda()
    T, H, D = k.shape
    st = torch.cuda.current_stream().cuda_stream
    check(L.b200_rope_norm_f16(k.data_ptr(), D * 2, H * D * 2, k.data_ptr(), D * 2, H * D * 2, D, H, T, D, shift.data_ptr(), None, 500000.0, 1.0, 1.0, st))
    torch.cuda.synchronize()
    got = k.cpu().numpy().view(np.uint16)
    want = golden["rope_f16"]
    gf, wf = got.view(np.float16).astype(np.float32), want.view(np.float16).astype(np.float32)
    assert (got == want).mean() > 0.995
    assert np.all(np.abs(gf - wf) <= np.spacing(np.abs(wf).astype(np.float16)).astype(np.float32))
    assert np.array_equal(got[r["shift"] == 0], r["kf16"][r["shift"] == 0])
    # defragmentation move: rows [5, 9) of a strided cache view to rows [0, 4)
    cache = torch.arange(12 * 64, dtype=torch.int16, device="cuda").view(12, 64)
    before = cache.cpu().numpy().copy()
    check(L.b200_cpy_f16_f16(cache[5:].data_ptr(), 128, cache.data_ptr(), 128, 64, 4, st))
    torch.cuda.synchronize()
    after = cache.cpu().numpy()
    assert np.array_equal(after[:4], before[5:9]) and np.array_equal(after[4:], before[4:])


def test_argmax_rows_first_maximum_on_aligned_and_unaligned_rows():
    """The greedy choice: lowest index among equal maxima, on rows that start on and off 16-byte boundaries, with
    lengths that are and are not multiples of four, at the vocabulary size and below one pass of the CTA."""
    from cactus_b200 import ops
    rng = np.random.default_rng(5)
    for d, stride, off in ((128256, 128256, 0), (32000, 32004, 0), (32001, 32003, 1), (4099, 4099, 3), (37, 40, 2), (1, 4, 0)):
        rows = 5
        buf = rng.standard_normal(off + rows * stride).astype(np.float32)
        a = buf[off:off + rows * stride].reshape(rows, stride)[:, :d]
        a[1, :] = -np.inf                                  # nothing beats the start value: index 0
        if d > 8:
            a[2, [d - 1, d // 2, 7]] = 9.0                 # equal maxima: the first one
            a[3, d - 1] = 11.0                             # the maximum in the ragged tail
            a[4, :] = np.round(a[4, :])                    # many ties
        t = dev(buf)[off:off + rows * stride].view(rows, stride)[:, :d]
        got = host(ops.argmax_rows(t))
        assert np.array_equal(got, a.argmax(-1).astype(np.int32)), (d, stride, off, got, a.argmax(-1))

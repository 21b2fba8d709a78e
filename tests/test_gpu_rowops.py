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

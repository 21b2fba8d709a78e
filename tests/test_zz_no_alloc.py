"""The allocation-free mul_mat entry point, b200_mul_mat_q_noalloc.

It exists for callers that cannot give the library a scratch buffer or let it allocate one -- a host with a fixed
device-memory budget, a plug-in inside a process whose allocator owns the GPU's memory -- and keeps the quantised
activations in an array built into the library instead.  The test calls it through the C ABI twice in a row, with
different inputs (the array is shared between calls and still holds the first call's data during the second), and
checks each result against the ordinary entry point, which takes caller-provided scratch.  It also checks that sizes
beyond the built-in array are refused.  This file sorts last on purpose: a run that stops at the first failure has
then already run every other test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_noalloc_matches_the_scratch_taking_entry_point_twice_in_a_row():
    from cactus_b200 import ops
    from cactus_b200._lib import check, lib
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(11)
    for wtype, bb in ((2, 18), (8, 34)):
        M, K = 272, 2048
        blocks = torch.randint(0, 256, (M, K // 32 * bb), dtype=torch.uint8, device="cuda", generator=g)
        blocks.view(M, K // 32, bb)[:, :, 1] = 0x1C          # fp16 scales around 2^-8, finite
        w = ops.QWeight.from_blocks(wtype, K, M, blocks)
        for call, N in enumerate((5, 1)):                    # two calls back to back; the second is smaller than the first
            x = torch.randn((N, K), device="cuda", generator=g) * (1.0 + call)
            want = ops.mul_mat(w, x)                         # b200_mul_mat_q with scratch owned by the caller
            got = torch.full((N, M), float("nan"), device="cuda")
            before = torch.cuda.memory_allocated()
            check(L.b200_mul_mat_q_noalloc(wtype, w.data.data_ptr(), K, M, x.data_ptr(), K * 4, N, got.data_ptr(), M * 4, 0,
                                           torch.cuda.current_stream().cuda_stream))
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated() == before
            a, b = got.cpu().numpy(), want.cpu().numpy()
            assert np.isfinite(a).all()
            # the same kernels run on the same quantised data: equal, and in any case within the mul_mat tolerance
            assert np.abs(a - b).max() / np.abs(b).max() < 1e-3
            assert np.array_equal(a, b)


@pytest.mark.parametrize("wtype,bb", [(2, 18), (8, 34)])
@pytest.mark.parametrize("K,N", [(32768, 8), (2048 + 3 * 32, 3), (2048 + 32, 8), (32768, 1)])
def test_noalloc_at_its_limits_and_with_ragged_block_counts(wtype, bb, K, N):
    """The largest size the built-in array admits (8 columns of 32768 values) and rows whose block count is not a
    multiple of the 4-block groups of the tiled layout.  For 3 and more columns the ordinary entry point may split K
    through its workspace and this one may not, so the comparison is the mul_mat tolerance, against the oracle too.
    The device's free memory (cudaMemGetInfo) must not move across the call."""
    from cactus_b200 import ops
    from cactus_b200._lib import check, lib
    from oracle.binding import Oracle
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(K + N)
    M = 80
    blocks = torch.randint(0, 256, (M, K // 32 * bb), dtype=torch.uint8, device="cuda", generator=g)
    blocks.view(M, K // 32, bb)[:, :, 1] = 0x1C
    w = ops.QWeight.from_blocks(wtype, K, M, blocks)
    x = torch.randn((N, K), device="cuda", generator=g)
    want = ops.mul_mat(w, x)
    got = torch.full((N, M), float("nan"), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    check(L.b200_mul_mat_q_noalloc(wtype, w.data.data_ptr(), K, M, x.data_ptr(), K * 4, N, got.data_ptr(), M * 4, 0, st))   # first use on this device
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    got.fill_(float("nan"))
    check(L.b200_mul_mat_q_noalloc(wtype, w.data.data_ptr(), K, M, x.data_ptr(), K * 4, N, got.data_ptr(), M * 4, 0, st))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    a, b = got.cpu().numpy(), want.cpu().numpy()
    assert np.isfinite(a).all()
    assert np.abs(a - b).max() / np.abs(b).max() < 1e-3
    ref, _ = Oracle().mul_mat(wtype, blocks.cpu().numpy(), x.cpu().numpy(), 0)
    assert np.abs(a - ref).max() / np.abs(ref).max() < 1e-3


def test_noalloc_refuses_sizes_beyond_the_built_in_array():
    from cactus_b200._lib import lib
    L = lib()
    x = torch.zeros(64, device="cuda")
    rc = L.b200_mul_mat_q_noalloc(2, x.data_ptr(), 4096, 16, x.data_ptr(), 4096 * 4, 9, x.data_ptr(), 64, 0, None)
    assert rc == -1 and b"at most 8 columns" in L.b200_last_error()
    rc = L.b200_mul_mat_q_noalloc(2, x.data_ptr(), 65536, 16, x.data_ptr(), 65536 * 4, 1, x.data_ptr(), 64, 0, None)
    assert rc == -1 and b"at most 32768" in L.b200_last_error()

"""K2-K4 on the GPU: Q4_0 / Q8_0 mul_mat against the oracle and the golden vectors.

Integer block dots: exact.  Final floats: max|gpu - ref| / max|ref| <= 1e-3 (the float summation order
over blocks differs from the reference's AVX2 order, so bit equality is not expected).
"""
import numpy as np
import pytest
import torch

import inputs
from gpu_util import dev, host, rel_max_err
from oracle.binding import Q4_0, Q8_0

pytestmark = pytest.mark.gpu
TOL = 1e-3
NAMES = {Q4_0: "q4", Q8_0: "q8"}


@pytest.mark.parametrize("wtype", [Q4_0, Q8_0])
def test_block_dots_exact_vs_golden(golden, wtype):
    from cactus_b200 import ops
    xa = inputs.small_activations()
    w = ops.QWeight.from_blocks(wtype, 256, 24, golden["w" + NAMES[wtype]])
    assert np.array_equal(host(ops.block_dots(w, dev(xa))), golden["dots_" + NAMES[wtype]])


@pytest.mark.parametrize("wtype", [Q4_0, Q8_0])
def test_small_mul_mat_vs_golden(golden, wtype):
    from cactus_b200 import ops
    xa = inputs.small_activations()
    w = ops.QWeight.from_blocks(wtype, 256, 24, golden["w" + NAMES[wtype]])
    got = host(ops.mul_mat(w, dev(xa)))
    assert rel_max_err(got, golden["mm_" + NAMES[wtype]]) < TOL


@pytest.mark.parametrize("wtype", [Q4_0, Q8_0])
@pytest.mark.parametrize("N", [1, 2, 3, 7, 8, 9, 15, 16, 17, 31, 33, 63, 64, 65])
def test_column_counts_vs_oracle(oracle, wtype, N):
    """Every kernel variant boundary: dp4a kernel (1..8), 32- and 64-column tensor-core tiles, ragged tails."""
    from cactus_b200 import ops
    M, K = 80, 512          # M not a multiple of the 64-row CTA tile
    rng = np.random.default_rng(1000 + N)
    wq = oracle.quantize_weights(wtype, (rng.standard_normal((M, K)) * 0.02).astype(np.float32))
    x = rng.standard_normal((N, K)).astype(np.float32)
    ref, _ = oracle.mul_mat(wtype, wq, x)
    w = ops.QWeight.from_blocks(wtype, K, M, wq)
    got = host(ops.mul_mat(w, dev(x)))
    assert got.shape == (N, M)
    assert rel_max_err(got, ref) < TOL
    # and the integer dots behind it are exact
    assert np.array_equal(host(ops.block_dots(w, dev(x))), oracle.block_dots(wtype, wq, oracle.quantize_q8_0(x), K))


@pytest.mark.parametrize("wtype", [Q4_0, Q8_0])
@pytest.mark.parametrize("shape", [(33, 32, 1), (17, 64, 5), (1, 96, 12), (130, 160, 40), (16, 14336, 3), (48, 14336, 20)])
def test_odd_shapes_vs_oracle(oracle, wtype, shape):
    """Rows not a multiple of 16, blocks not a multiple of 4 (padding paths), long K (split-K path)."""
    from cactus_b200 import ops
    M, K, N = shape
    rng = np.random.default_rng(M * 3 + K + N)
    wq = oracle.quantize_weights(wtype, (rng.standard_normal((M, K)) * 0.02).astype(np.float32))
    x = rng.standard_normal((N, K)).astype(np.float32)
    ref, _ = oracle.mul_mat(wtype, wq, x)
    got = host(ops.mul_mat(ops.QWeight.from_blocks(wtype, K, M, wq), dev(x)))
    assert rel_max_err(got, ref) < TOL


def test_strided_activations_and_output(oracle):
    """src1 rows with nb11 != row size and a dst with a row stride, as views in a graph produce them."""
    from cactus_b200 import ops
    M, K, N = 64, 256, 12
    rng = np.random.default_rng(9)
    wq = oracle.quantize_weights(Q4_0, (rng.standard_normal((M, K)) * 0.02).astype(np.float32))
    big = rng.standard_normal((N, 3 * K)).astype(np.float32)
    ref, _ = oracle.mul_mat(Q4_0, wq, np.ascontiguousarray(big[:, K:2 * K]))
    out = torch.full((N, 2 * M), 7.0, device="cuda")
    ops.mul_mat(ops.QWeight.from_blocks(Q4_0, K, M, wq), dev(big)[:, K:2 * K], out=out[:, :M])
    o = host(out)
    assert rel_max_err(o[:, :M], ref) < TOL
    assert (o[:, M:] == 7.0).all()


def test_zero_and_degenerate_blocks(oracle):
    from cactus_b200 import ops
    M, K = 32, 128
    w = np.zeros((M, K), np.float32)
    w[3, 40] = 0.5
    x = np.zeros((2, K), np.float32)
    x[1, 40] = -2.0
    wq = oracle.quantize_weights(Q4_0, w)
    ref, _ = oracle.mul_mat(Q4_0, wq, x)
    got = host(ops.mul_mat(ops.QWeight.from_blocks(Q4_0, K, M, wq), dev(x)))
    assert np.isfinite(got).all() and np.abs(got - ref).max() <= 1e-6


@pytest.mark.parametrize("N", [1, 8, 512])
def test_config1_vs_golden(oracle, golden, N):
    """Config 1: Q4_0 [4096 x 4096] x f32 [4096 x N], N in {1, 8, 512}, seed 0."""
    from cactus_b200 import ops
    wq = oracle.quantize_weights(Q4_0, inputs.cfg1_weights())
    assert inputs.checksum(wq) == int(golden["cfg1_wq_crc"][0])
    got = host(ops.mul_mat(ops.QWeight.from_blocks(Q4_0, 4096, 4096, wq), dev(inputs.cfg1_activations(N))))
    sample = golden[f"cfg1_n{N}_sample"]
    mine = got[:, ::inputs.CFG1_SAMPLE_STRIDE] if N > 8 else got
    scale = float(np.abs(sample).max())
    assert np.abs(mine - sample).max() / scale < TOL
    s, sa = golden[f"cfg1_n{N}_sum"]
    assert abs(got.astype(np.float64).sum() - s) / sa < 1e-5     # checksum over the whole output
    assert abs(np.abs(got).astype(np.float64).sum() - sa) / sa < 1e-5


def test_head_shape_q8_0_vs_golden(oracle, golden):
    from cactus_b200 import ops
    wq = oracle.quantize_weights(Q8_0, inputs.head_weights())
    got = host(ops.mul_mat(ops.QWeight.from_blocks(Q8_0, 2048, 512, wq), dev(inputs.head_activations())))
    assert rel_max_err(got, golden["head_q8"]) < TOL


def test_kernels_agree_column_by_column():
    """Size-independent property at full size: a column of the N=512 tensor-core product equals the N=1
    dp4a product of that column (same integer dots, different float order)."""
    from cactus_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(3)
    M, K = 14336, 4096
    blocks = torch.randint(0, 256, (M, K // 32 * 18), dtype=torch.uint8, device="cuda", generator=g)
    blocks.view(M, K // 32, 18)[:, :, 1] = (blocks.view(M, K // 32, 18)[:, :, 1] & 0x03) | 0x18  # fp16 scales ~ 2^-9..2^-8
    w = ops.QWeight.from_blocks(2, K, M, blocks)
    x = torch.randn((512, K), device="cuda", generator=g)
    big = ops.mul_mat(w, x)
    for n in (0, 77, 511):
        one = ops.mul_mat(w, x[n:n + 1])
        assert rel_max_err(host(big[n:n + 1]), host(one)) < 1e-4
    eight = ops.mul_mat(w, x[8:16])
    assert rel_max_err(host(big[8:16]), host(eight)) < 1e-4


@pytest.mark.parametrize("wtype", [Q4_0, Q8_0])
def test_weight_cat_and_row_slice(oracle, wtype):
    """Stacking weights row-wise (wq/wk/wv, gate/up as one mul_mat) and cutting row ranges (row split) are byte-range
    operations on the tiled layout: both must reproduce the reference block streams exactly."""
    from cactus_b200 import ops
    K = 288   # 9 blocks: not a multiple of the 4-block tile
    rng = np.random.default_rng(77)
    parts = [np.asarray(oracle.quantize_weights(wtype, (rng.standard_normal((M, K)) * 0.02).astype(np.float32))) for M in (48, 32, 20)]
    ws = [ops.QWeight.from_blocks(wtype, K, p.shape[0], p) for p in parts]
    cat = ops.QWeight.cat(ws)
    assert cat.M == 100
    assert np.array_equal(host(cat.to_blocks()), np.concatenate([p.reshape(p.shape[0], -1) for p in parts]))
    mid = cat.row_slice(48, 80)
    assert np.array_equal(host(mid.to_blocks()), parts[1].reshape(32, -1))
    tail = cat.row_slice(80, 100)
    assert np.array_equal(host(tail.to_blocks()), parts[2].reshape(20, -1))
    x = rng.standard_normal((5, K)).astype(np.float32)
    whole = host(ops.mul_mat(cat, dev(x)))
    for w, lo in zip(ws, (0, 48, 80)):
        assert rel_max_err(whole[:, lo:lo + w.M], host(ops.mul_mat(w, dev(x)))) < 1e-6


@pytest.mark.parametrize("K,Ms,N", [(4096, [14336, 14336], 64), (4096, [4096, 1024, 1024], 64), (512, [256, 128], 20), (1024, [128, 128, 80], 33),
                                    (2048 + 96, [384, 256], 9), (512, [100, 128], 16), (512, [256, 128], 2)])
def test_several_weights_in_one_launch_match_the_separate_products(K, Ms, N):
    """b200_mul_mat_q_prequant_multi: separate weight tensors and separate destinations, one launch (stream-K, cluster
    split-K, plain grid and the split-K reduction all occur among these shapes; the last two fall back to one product
    after the other).  The work is dealt out differently than for the single products, so the fp32 sums may come in
    another order: equal to 1e-5 of the largest value, and within the mul_mat tolerance of the oracle."""
    import ctypes as C

    from cactus_b200 import ops
    from cactus_b200._lib import check, lib
    from cactus_b200.engine import random_blocks
    L = lib()
    gen = torch.Generator(device="cuda").manual_seed(K + N + len(Ms))
    ws = [ops.QWeight.from_blocks(2, K, M, random_blocks(2, M, K, gen)) for M in Ms]
    x = torch.randn((N, K), device="cuda", generator=gen)
    act = torch.empty(L.b200_act_bytes(K, N), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    check(L.b200_quantize_activations(x.data_ptr(), K * 4, K, N, act.data_ptr(), act.numel(), 0, st))
    wsp = torch.empty(max(256, L.b200_mul_mat_workspace_bytes(2, K, sum(Ms), N)), dtype=torch.uint8, device="cuda")
    stride = max(Ms)                                              # one row stride for all destinations, as the entry point asks
    want, got = [], []
    for w in ws:
        o = torch.zeros((N, stride), device="cuda")
        check(L.b200_mul_mat_q_prequant(2, w.data.data_ptr(), K, w.M, act.data_ptr(), N, o.data_ptr(), stride * 4, wsp.data_ptr(), wsp.numel(), st))
        want.append(o)
        got.append(torch.full((N, stride), float("nan"), device="cuda"))
    wp = (C.c_void_p * len(ws))(*[w.data.data_ptr() for w in ws])
    mp = (C.c_int64 * len(ws))(*Ms)
    dp = (C.c_void_p * len(ws))(*[g.data_ptr() for g in got])
    check(L.b200_mul_mat_q_prequant_multi(2, len(ws), wp, mp, K, act.data_ptr(), N, dp, stride * 4, wsp.data_ptr(), wsp.numel(), st))
    torch.cuda.synchronize()
    for w, a, b in zip(ws, got, want):
        a, b = a[:, :w.M].cpu().numpy(), b[:, :w.M].cpu().numpy()
        assert np.isfinite(a).all()
        assert np.abs(a - b).max() <= 1e-5 * np.abs(b).max()
    if K * sum(Ms) <= 1 << 21:                                    # the oracle on the small cases
        from oracle.binding import Oracle
        o = Oracle()
        for w, a in zip(ws, got):
            ref, _ = o.mul_mat(2, w.to_blocks().cpu().numpy(), x.cpu().numpy(), 0)
            assert np.abs(a[:, :w.M].cpu().numpy() - ref).max() / np.abs(ref).max() < 1e-3

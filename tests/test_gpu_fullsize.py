"""The hot ops at the benchmark's full sizes (8B architecture, 64 sequences, the 57314-cell ragged cache), checked
through constructions whose pieces are pinned to the oracle at small sizes:

* mul_mat: the product must equal (dequantised weights) x (dequantised Q8_0 activations) formed in float64 -- with the
  activation blocks taken from the library's own quantiser, which the small-size tests hold bit-exact to the reference;
* flash attention: every token against a float64 softmax over its own sequence's cells;
* the fused norm at 64 x 4096 against the chain of separate ops, bit for bit.

Tolerances are the op tolerances of the small-size tests (1e-3 / 2e-3 of the largest output)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dequant_q4_0(blocks: torch.Tensor, M: int, K: int) -> torch.Tensor:
    b = blocks.view(M, K // 32, 18)
    d = b[..., :2].contiguous().view(torch.float16).to(torch.float64)             # [M, nb, 1]
    qs = b[..., 2:]
    lo, hi = (qs & 0xF).to(torch.float64) - 8.0, (qs >> 4).to(torch.float64) - 8.0
    return (torch.cat([lo, hi], dim=-1) * d).reshape(M, K)


def _dequant_q8_0(blocks: torch.Tensor, N: int, K: int) -> torch.Tensor:
    b = blocks.view(N, K // 32, 34)
    d = b[..., :2].contiguous().view(torch.float16).to(torch.float64)
    return (b[..., 2:].contiguous().view(torch.int8).to(torch.float64) * d).reshape(N, K)


@pytest.mark.parametrize("shape", [(4096, 14336), (14336, 4096), (4096, 6144)])
def test_mul_mat_full_size(shape):
    from cactus_b200 import ops
    from cactus_b200.engine import random_blocks
    K, M = shape
    N = 64
    gen = torch.Generator(device="cuda").manual_seed(K + M)
    blocks = random_blocks(ops.Q4_0, M, K, gen)
    x = torch.randn((N, K), device="cuda", generator=gen)
    got = ops.mul_mat(ops.QWeight.from_blocks(ops.Q4_0, K, M, blocks), x).to(torch.float64)
    xq = ops.quantize_row_q8_0(x)
    want = _dequant_q8_0(xq, N, K) @ _dequant_q4_0(blocks, M, K).T
    err = float((got - want).abs().max() / want.abs().max())
    assert err < 1e-3, err


def test_flash_attn_full_size_ragged():
    from cactus_b200 import ops
    from cactus_b200._lib import check, lib
    from cactus_b200.workloads import prompt_lengths
    L = lib()
    lens = torch.from_numpy(prompt_lengths()[0]).cuda()
    n_seq, H, Hkv, D = int(lens.numel()), 32, 8, 128
    total = int(lens.sum())
    n_cells = (total + 255) // 256 * 256
    gen = torch.Generator(device="cuda").manual_seed(3)
    k = torch.randn((n_cells, Hkv, D), device="cuda", generator=gen).half()
    v = torch.randn((n_cells, Hkv, D), device="cuda", generator=gen).half()
    q = torch.randn((n_seq, H, D), device="cuda", generator=gen)
    ends = torch.cumsum(lens, 0)
    cells = torch.arange(n_cells, device="cuda")
    owner = torch.searchsorted(ends, cells, right=True)
    cell_seq = owner.to(torch.int32)
    cell_seq[cells >= total] = -1
    cell_pos = (cells - (ends - lens)[owner.clamp(max=n_seq - 1)]).to(torch.int32)
    tok_pos, tok_seq = (lens - 1).to(torch.int32), torch.arange(n_seq, dtype=torch.int32, device="cuda")
    mask = torch.empty((64, n_cells), dtype=torch.float16, device="cuda")
    check(L.b200_kq_mask_build(cell_pos.data_ptr(), cell_seq.data_ptr(), n_cells, tok_pos.data_ptr(), tok_seq.data_ptr(), n_seq, mask.data_ptr(),
                               n_cells * 2, torch.cuda.current_stream().cuda_stream))
    got = ops.flash_attn_ext(q, k, v, mask, D ** -0.5).to(torch.float64)
    worst = 0.0
    starts = (ends - lens).tolist()
    for s in range(n_seq):
        ks = k[starts[s]:starts[s] + int(lens[s])].to(torch.float64)     # [ctx, Hkv, D]
        vs = v[starts[s]:starts[s] + int(lens[s])].to(torch.float64)
        qs = q[s].to(torch.float16).to(torch.float64).view(Hkv, H // Hkv, D)   # the reference rounds q to f16
        sc = torch.einsum("hgd,chd->hgc", qs, ks) * D ** -0.5
        p = torch.softmax(sc, dim=-1)
        o = torch.einsum("hgc,chd->hgd", p, vs).reshape(H, D)
        worst = max(worst, float((got[s] - o).abs().max() / o.abs().max()))
    assert worst < 2e-3, worst


def test_fused_norm_full_size():
    from cactus_b200._lib import check, lib
    L = lib()
    N, d = 64, 4096
    gen = torch.Generator(device="cuda").manual_seed(5)
    x0 = torch.randn((N, d), device="cuda", generator=gen)
    r = torch.randn((N, d), device="cuda", generator=gen)
    w = torch.randn(d, device="cuda", generator=gen)
    st = torch.cuda.current_stream().cuda_stream
    n = L.b200_act_bytes(d, N)
    sa, sb = torch.zeros(n, dtype=torch.uint8, device="cuda"), torch.zeros(n, dtype=torch.uint8, device="cuda")
    xa = x0.clone()
    check(L.b200_add(xa.data_ptr(), r.data_ptr(), xa.data_ptr(), d, N, N, st))
    h = torch.empty_like(xa)
    check(L.b200_rms_norm(xa.data_ptr(), d * 4, w.data_ptr(), h.data_ptr(), d * 4, d, N, 1e-5, st))
    check(L.b200_quantize_activations(h.data_ptr(), d * 4, d, N, sa.data_ptr(), n, 0, st))
    xb = x0.clone()
    check(L.b200_add_rms_norm_quantize(xb.data_ptr(), d * 4, r.data_ptr(), d * 4, w.data_ptr(), None, 0, d, N, 1e-5, sb.data_ptr(), n, 0, st))
    torch.cuda.synchronize()
    assert torch.equal(xa.view(torch.int32), xb.view(torch.int32)) and torch.equal(sa, sb)

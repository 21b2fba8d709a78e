"""The fused layer ops against the chain of separate ops they replace: every output bit for bit (the quantised
activation scratch, the updated residual stream, the rotated q, the f16 cache rows)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _st():
    return torch.cuda.current_stream().cuda_stream


def _scratch(L, K, N):
    n = L.b200_act_bytes(K, N)
    return torch.full((n,), 0xAB, dtype=torch.uint8, device="cuda"), torch.full((n,), 0xAB, dtype=torch.uint8, device="cuda")


@pytest.mark.parametrize("N", [1, 5, 8, 9, 64])
@pytest.mark.parametrize("d", [256, 160])
@pytest.mark.parametrize("with_residual", [False, True])
def test_add_rms_norm_quantize(N, d, with_residual):
    from cactus_b200._lib import check, lib
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(N * 1000 + d)
    x0 = torch.randn((N, d), device="cuda", generator=g)
    r = torch.randn((N, d), device="cuda", generator=g)
    w = torch.randn(d, device="cuda", generator=g)
    eps = 1e-5
    # separate ops
    xa = x0.clone()
    if with_residual:
        check(L.b200_add(xa.data_ptr(), r.data_ptr(), xa.data_ptr(), d, N, N, _st()))
    h = torch.empty_like(xa)
    check(L.b200_rms_norm(xa.data_ptr(), d * 4, w.data_ptr(), h.data_ptr(), d * 4, d, N, eps, _st()))
    sa, sb = _scratch(L, d, N)
    check(L.b200_quantize_activations(h.data_ptr(), d * 4, d, N, sa.data_ptr(), sa.numel(), 0, _st()))
    # fused
    xb = x0.clone()
    hb = torch.empty_like(xb)
    check(L.b200_add_rms_norm_quantize(xb.data_ptr(), d * 4, r.data_ptr() if with_residual else None, d * 4, w.data_ptr(), hb.data_ptr(), d * 4,
                                       d, N, eps, sb.data_ptr(), sb.numel(), 0, _st()))
    torch.cuda.synchronize()
    assert torch.equal(xa.view(torch.int32), xb.view(torch.int32))
    assert torch.equal(h.view(torch.int32), hb.view(torch.int32))
    assert torch.equal(sa, sb)


@pytest.mark.parametrize("N", [1, 7, 64])
@pytest.mark.parametrize("K", [512, 160])
def test_silu_mul_quantize(N, K):
    from cactus_b200._lib import check, lib
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(N + K)
    gate = torch.randn((N, K), device="cuda", generator=g) * 3
    up = torch.randn((N, K), device="cuda", generator=g)
    act = torch.empty_like(gate)
    check(L.b200_silu(gate.data_ptr(), up.data_ptr(), act.data_ptr(), N * K, _st()))
    sa, sb = _scratch(L, K, N)
    check(L.b200_quantize_activations(act.data_ptr(), K * 4, K, N, sa.data_ptr(), sa.numel(), 0, _st()))
    out = torch.empty_like(gate)
    check(L.b200_silu_mul_quantize(gate.data_ptr(), up.data_ptr(), K * 4, out.data_ptr(), K * 4, K, N, sb.data_ptr(), sb.numel(), 0, _st()))
    torch.cuda.synchronize()
    assert torch.equal(sa, sb)
    assert torch.equal(act.view(torch.int32), out.view(torch.int32))
    sb.fill_(0xAB)
    check(L.b200_silu_mul_quantize(gate.data_ptr(), up.data_ptr(), K * 4, None, 0, K, N, sb.data_ptr(), sb.numel(), 0, _st()))
    torch.cuda.synchronize()
    assert torch.equal(sa, sb)


@pytest.mark.parametrize("T", [1, 13])
def test_rope_store(T):
    from cactus_b200._lib import check, lib
    L = lib()
    D, H, Hkv, cells = 64, 4, 2, 32
    g = torch.Generator(device="cuda").manual_seed(T)
    q0 = torch.randn((T, H * D), device="cuda", generator=g)
    k0 = torch.randn((T, Hkv * D), device="cuda", generator=g)
    v0 = torch.randn((T, Hkv * D), device="cuda", generator=g)
    pos = torch.arange(5, 5 + T, dtype=torch.int32, device="cuda")
    slots = torch.randperm(cells, device="cuda", generator=g)[:T].to(torch.int32)
    kvd = Hkv * D
    # separate ops
    qa, ka = q0.clone(), k0.clone()
    kca = torch.zeros((cells, kvd), dtype=torch.float16, device="cuda")
    vca = torch.zeros_like(kca)
    check(L.b200_rope_norm(qa.data_ptr(), D * 4, H * D * 4, qa.data_ptr(), D * 4, H * D * 4, D, H, T, D, pos.data_ptr(), None, 500000.0, 1.0, 1.0, _st()))
    check(L.b200_rope_norm(ka.data_ptr(), D * 4, kvd * 4, ka.data_ptr(), D * 4, kvd * 4, D, Hkv, T, D, pos.data_ptr(), None, 500000.0, 1.0, 1.0, _st()))
    check(L.b200_set_rows_f16(ka.data_ptr(), kvd * 4, slots.data_ptr(), kca.data_ptr(), kvd * 2, kvd, T, _st()))
    check(L.b200_set_rows_f16(v0.data_ptr(), kvd * 4, slots.data_ptr(), vca.data_ptr(), kvd * 2, kvd, T, _st()))
    # fused
    qb = q0.clone()
    kcb = torch.zeros_like(kca)
    vcb = torch.zeros_like(kca)
    check(L.b200_rope_store(qb.data_ptr(), D * 4, H * D * 4, k0.data_ptr(), D * 4, kvd * 4, v0.data_ptr(), kvd * 4, D, H, Hkv, T, D, pos.data_ptr(), None,
                            500000.0, 1.0, 1.0, slots.data_ptr(), kcb.data_ptr(), kvd * 2, vcb.data_ptr(), kvd * 2, _st()))
    torch.cuda.synchronize()
    assert torch.equal(qa.view(torch.int32), qb.view(torch.int32))
    assert torch.equal(kca.view(torch.int16), kcb.view(torch.int16))
    assert torch.equal(vca.view(torch.int16), vcb.view(torch.int16))


@pytest.mark.parametrize("Nq,n_kv,H,Hkv,D", [(13, 1024, 8, 2, 128),     # ragged tokens, padding columns, one KV split
                                            (64, 2048, 32, 8, 128),    # the decode batch shape
                                            (2, 16384, 8, 2, 128),     # few tokens over a long cache: several KV splits + combine kernel
                                            (1, 4096, 32, 8, 128),     # one token (single-sequence decode): the engine's path for up to two tokens
                                            (9, 512, 4, 4, 64)])       # head size 64, no grouping
def test_flash_attn_quantised_output(Nq, n_kv, H, Hkv, D):
    """b200_flash_attn_ext_quant leaves exactly what the attention followed by the activation quantiser leaves."""
    from cactus_b200._lib import check, lib
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(Nq * 7 + n_kv)
    q = torch.randn((Nq, H, D), device="cuda", generator=g)
    k = torch.randn((n_kv, Hkv, D), device="cuda", generator=g).half()
    v = torch.randn((n_kv, Hkv, D), device="cuda", generator=g).half()
    # every token sees its own random prefix of the cache
    lens = torch.randint(1, n_kv + 1, (Nq,), device="cuda", generator=g)
    mask = torch.full((Nq, n_kv), float("-inf"), dtype=torch.float16, device="cuda")
    mask[torch.arange(n_kv, device="cuda")[None, :] < lens[:, None]] = 0
    index = torch.empty(L.b200_mask_index_bytes(Nq, n_kv), dtype=torch.uint8, device="cuda")
    check(L.b200_mask_index_build(mask.data_ptr(), n_kv * 2, Nq, n_kv, index.data_ptr(), index.numel(), _st()))
    scratch = torch.empty(max(256, L.b200_flash_attn_scratch_bytes(D, H, Hkv, Nq, n_kv)), dtype=torch.uint8, device="cuda")
    args = (D, H, Hkv, Nq, n_kv, q.data_ptr(), H * D * 4, D * 4, k.data_ptr(), Hkv * D * 2, D * 2, v.data_ptr(), Hkv * D * 2, D * 2,
            mask.data_ptr(), n_kv * 2, index.data_ptr(), D ** -0.5, 0.0, 0.0)
    out = torch.empty((Nq, H * D), device="cuda")
    check(L.b200_flash_attn_ext_indexed(*args, out.data_ptr(), scratch.data_ptr(), scratch.numel(), _st()))
    sa, sb = _scratch(L, H * D, Nq)
    check(L.b200_quantize_activations(out.data_ptr(), H * D * 4, H * D, Nq, sa.data_ptr(), sa.numel(), 0, _st()))
    out2 = torch.empty_like(out)
    check(L.b200_flash_attn_ext_quant(*args, out2.data_ptr(), sb.data_ptr(), sb.numel(), 0, scratch.data_ptr(), scratch.numel(), _st()))
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int32), out2.view(torch.int32))
    assert torch.equal(sa, sb)
    sb.fill_(0xAB)
    check(L.b200_flash_attn_ext_quant(*args, None, sb.data_ptr(), sb.numel(), 0, scratch.data_ptr(), scratch.numel(), _st()))
    torch.cuda.synchronize()
    assert torch.equal(sa, sb)

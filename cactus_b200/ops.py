"""Host-side mirror of the ggml ops the backend serves, over the C ABI.

Names and argument meaning follow the reference's op builders (cactus/ggml.h): ``mul_mat(w, x)``,
``flash_attn_ext(q, k, v, mask, scale, max_bias, logit_softcap)``, ``rms_norm``, ``rope_ext``, ``cpy``,
``get_rows``, ``silu``, ``add``, ``mul``.  Tensors are torch CUDA tensors, used only as device memory
and for the current stream; every computation is a call into libcactus_b200.so.
"""
from __future__ import annotations

import numpy as np
import torch

from ._lib import B200Error, check, lib

Q4_0, Q8_0 = 2, 8
Q8_AVX2, Q8_SCALAR = 0, 1
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise B200Error("cactus_b200 ops need CUDA tensors; there is no CPU path")


class QWeight:
    """A quantised weight tensor [K, M] (ggml ne = [K, M]) resident on the device in the tiled layout."""

    def __init__(self, wtype: int, K: int, M: int, data: torch.Tensor, row0: int = 0):
        self.wtype, self.K, self.M, self.data = wtype, K, M, data
        self.row0 = row0   # first row of this weight within the tensor it was cut from (row split)
        self.parts = None  # row split of a stacked weight: [(rows, first column in the joined output), ...] of this rank's pieces

    @staticmethod
    def from_blocks(wtype: int, K: int, M: int, blocks, device="cuda") -> "QWeight":
        """blocks: uint8 [M, K/32*block_bytes] in the reference's row-major block layout (numpy or torch)."""
        L = lib()
        if isinstance(blocks, np.ndarray):
            blocks = torch.from_numpy(np.ascontiguousarray(blocks))
        src = blocks.to(device=device, dtype=torch.uint8).contiguous()
        assert src.numel() == M * (K // 32) * BLOCK_BYTES[wtype]
        nbytes = L.b200_weight_bytes(wtype, K, M)
        if nbytes == 0:
            raise B200Error("unsupported weight shape/type")
        data = torch.empty(nbytes, dtype=torch.uint8, device=device)
        check(L.b200_weight_upload(wtype, K, M, src.data_ptr(), data.data_ptr(), 0, M, _stream()))
        torch.cuda.current_stream().synchronize()  # src may be freed by the caller
        return QWeight(wtype, K, M, data)

    def row_slice(self, r0: int, r1: int) -> "QWeight":
        """Rows [r0, r1) as a weight of its own (a copy).  Tiles are stored row-tile-major, so a slice on 16-row
        boundaries is one byte range of the quant plane plus one of the scale plane."""
        assert 0 <= r0 < r1 <= self.M and r0 % 16 == 0 and (r1 % 16 == 0 or r1 == self.M), "row slices start and end on 16-row tiles"
        n_rt, n_bg = (self.M + 15) // 16, (self.K // 32 + 3) // 4
        tile = 1024 if self.wtype == Q4_0 else 2048
        t0, t1 = r0 // 16, (r1 + 15) // 16
        q = self.data[t0 * n_bg * tile:t1 * n_bg * tile]
        d = self.data[n_rt * n_bg * tile + t0 * n_bg * 128:n_rt * n_bg * tile + t1 * n_bg * 128]
        return QWeight(self.wtype, self.K, r1 - r0, torch.cat([q, d]), row0=self.row0 + r0)

    @staticmethod
    def cat(parts: list) -> "QWeight":
        """The rows of several weights with the same K and type stacked into one weight (a copy): one mul_mat then
        yields all their products side by side.  Every part but the last must have a multiple of 16 rows."""
        w0 = parts[0]
        assert all(p.K == w0.K and p.wtype == w0.wtype for p in parts) and all(p.M % 16 == 0 for p in parts[:-1])
        n_bg = (w0.K // 32 + 3) // 4
        tile = 1024 if w0.wtype == Q4_0 else 2048
        qs = [p.data[:((p.M + 15) // 16) * n_bg * tile] for p in parts]
        ds = [p.data[((p.M + 15) // 16) * n_bg * tile:] for p in parts]
        return QWeight(w0.wtype, w0.K, sum(p.M for p in parts), torch.cat(qs + ds))

    def to_blocks(self) -> torch.Tensor:
        L = lib()
        out = torch.empty((self.M, self.K // 32 * BLOCK_BYTES[self.wtype]), dtype=torch.uint8, device=self.data.device)
        check(L.b200_weight_download(self.wtype, self.K, self.M, self.data.data_ptr(), out.data_ptr(), 0, self.M, _stream()))
        return out


def quantize_row_q8_0(x: torch.Tensor, variant: int = Q8_AVX2) -> torch.Tensor:
    """x f32 [N, K] (row stride free) -> uint8 [N, K/32*34]: the reference's block_q8_0 stream."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    N, K = x.shape
    out = torch.empty((N, K // 32 * 34), dtype=torch.uint8, device=x.device)
    check(lib().b200_quantize_q8_0(x.data_ptr(), x.stride(0) * 4, K, N, out.data_ptr(), variant, _stream()))
    return out


def mul_mat(w: QWeight, x: torch.Tensor, variant: int = Q8_AVX2, out: torch.Tensor | None = None,
            scratch: torch.Tensor | None = None) -> torch.Tensor:
    """dst[n, m] = sum_k W[m, k] x[n, k]  (ggml: dst = mul_mat(w, x) with ne = [M, N])."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] == w.K
    L = lib()
    N = x.shape[0]
    if out is None:
        out = torch.empty((N, w.M), dtype=torch.float32, device=x.device)
    need = L.b200_mul_mat_scratch_bytes(w.wtype, w.K, w.M, N)
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
    check(L.b200_mul_mat_q(w.wtype, w.data.data_ptr(), w.K, w.M, x.data_ptr(), x.stride(0) * 4, N, out.data_ptr(),
                           out.stride(0) * 4, scratch.data_ptr(), scratch.numel(), variant, _stream()))
    return out


def block_dots(w: QWeight, x: torch.Tensor, variant: int = Q8_AVX2) -> torch.Tensor:
    """int32 [N, M, K/32]: the exact per-block integer dot products behind mul_mat."""
    L = lib()
    N = x.shape[0]
    out = torch.empty((N, w.M, w.K // 32), dtype=torch.int32, device=x.device)
    act = torch.empty(L.b200_act_bytes(w.K, N), dtype=torch.uint8, device=x.device)
    check(L.b200_block_dots(w.wtype, w.data.data_ptr(), w.K, w.M, x.data_ptr(), x.stride(0) * 4, N, out.data_ptr(),
                            act.data_ptr(), act.numel(), variant, _stream()))
    return out


def flash_attn_ext(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor | None, scale: float,
                   max_bias: float = 0.0, logit_softcap: float = 0.0, n_kv: int | None = None, parity: bool = False) -> torch.Tensor:
    """q f32 [Nq, H, D]; k, v f16 [cells, Hkv, D] (the cache; the first n_kv cells are attended);
    mask f16 [>=Nq, n_kv] -> f32 [Nq, H, D].  ``parity=True`` runs the slow validation kernel that follows the
    reference's order of roundings (fp16 output accumulator) instead of the fast fp32-accumulating one."""
    _need_cuda(q, k, v, mask)
    L = lib()
    Nq, H, D = q.shape
    Hkv = k.shape[1]
    n_kv = k.shape[0] if n_kv is None else n_kv
    assert q.dtype == torch.float32 and k.dtype == torch.float16 and v.dtype == torch.float16
    assert q.stride(2) == 1 and k.stride(2) == 1 and v.stride(2) == 1
    out = torch.empty((Nq, H, D), dtype=torch.float32, device=q.device)
    need = L.b200_flash_attn_scratch_bytes(D, H, Hkv, Nq, n_kv)
    scratch = torch.empty(max(need, 256), dtype=torch.uint8, device=q.device)
    if mask is not None:
        assert mask.dtype == torch.float16 and mask.stride(1) == 1 and mask.shape[1] >= n_kv
    if parity:
        index = None
        if mask is not None:
            index = torch.empty(L.b200_mask_index_bytes(Nq, n_kv), dtype=torch.uint8, device=q.device)
            check(L.b200_mask_index_build(mask.data_ptr(), mask.stride(0) * 2, Nq, n_kv, index.data_ptr(), index.numel(), _stream()))
        check(L.b200_flash_attn_ext_parity(D, H, Hkv, Nq, n_kv, q.data_ptr(), q.stride(0) * 4, q.stride(1) * 4,
                                           k.data_ptr(), k.stride(0) * 2, k.stride(1) * 2, v.data_ptr(), v.stride(0) * 2, v.stride(1) * 2,
                                           mask.data_ptr() if mask is not None else None, mask.stride(0) * 2 if mask is not None else 0,
                                           index.data_ptr() if index is not None else None, scale, max_bias, logit_softcap, out.data_ptr(), _stream()))
        return out
    check(L.b200_flash_attn_ext(D, H, Hkv, Nq, n_kv, q.data_ptr(), q.stride(0) * 4, q.stride(1) * 4,
                                k.data_ptr(), k.stride(0) * 2, k.stride(1) * 2, v.data_ptr(), v.stride(0) * 2, v.stride(1) * 2,
                                mask.data_ptr() if mask is not None else None, mask.stride(0) * 2 if mask is not None else 0,
                                scale, max_bias, logit_softcap, out.data_ptr(), scratch.data_ptr(), scratch.numel(), _stream()))
    return out


def rms_norm(x: torch.Tensor, eps: float, weight: torch.Tensor | None = None) -> torch.Tensor:
    _need_cuda(x, weight)
    T, d = x.shape
    out = torch.empty((T, d), dtype=torch.float32, device=x.device)
    check(lib().b200_rms_norm(x.data_ptr(), x.stride(0) * 4, weight.data_ptr() if weight is not None else None, out.data_ptr(),
                              d * 4, d, T, eps, _stream()))
    return out


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    _need_cuda(a, b)
    a, b = a.contiguous(), b.contiguous()
    out = torch.empty_like(a)
    d = a.shape[-1]
    check(lib().b200_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), d, a.numel() // d, b.numel() // d, _stream()))
    return out


def mul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    _need_cuda(a, b)
    a, b = a.contiguous(), b.contiguous()
    out = torch.empty_like(a)
    d = a.shape[-1]
    check(lib().b200_mul(a.data_ptr(), b.data_ptr(), out.data_ptr(), d, a.numel() // d, b.numel() // d, _stream()))
    return out


def silu(a: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """SILU(a), or SILU(a) * b when b is given (the fused gate of the llama FFN)."""
    _need_cuda(a, b)
    a = a.contiguous()
    out = torch.empty_like(a)
    check(lib().b200_silu(a.data_ptr(), b.contiguous().data_ptr() if b is not None else None, out.data_ptr(), a.numel(), _stream()))
    return out


def rope_ext(x: torch.Tensor, pos: torch.Tensor, n_dims: int, freq_base: float, freq_scale: float = 1.0,
             attn_factor: float = 1.0, freq_factors: torch.Tensor | None = None) -> torch.Tensor:
    """x f32 [T, H, D], pos int32 [T]; mode 0 (adjacent pairs)."""
    _need_cuda(x, pos)
    T, H, D = x.shape
    assert x.stride(2) == 1 and pos.dtype == torch.int32
    out = torch.empty((T, H, D), dtype=torch.float32, device=x.device)
    check(lib().b200_rope_norm(x.data_ptr(), x.stride(1) * 4, x.stride(0) * 4, out.data_ptr(), D * 4, H * D * 4, D, H, T, n_dims,
                               pos.data_ptr(), freq_factors.data_ptr() if freq_factors is not None else None, freq_base,
                               freq_scale, attn_factor, _stream()))
    return out


def cpy(x: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """CPY of f32 rows into an f16 or f32 destination (e.g. a slice of the KV cache)."""
    _need_cuda(x, dst)
    T, d = x.shape
    assert dst.shape == x.shape and x.stride(1) == 1 and dst.stride(1) == 1
    fn = lib().b200_cpy_f32_f16 if dst.dtype == torch.float16 else lib().b200_cpy_f32_f32
    check(fn(x.data_ptr(), x.stride(0) * 4, dst.data_ptr(), dst.stride(0) * dst.element_size(), d, T, _stream()))
    return dst


def get_rows(table, ids: torch.Tensor) -> torch.Tensor:
    """table: QWeight [d, rows] or f32 tensor [rows, d]; ids int32 [n] -> f32 [n, d]."""
    _need_cuda(ids)
    n = ids.numel()
    if isinstance(table, QWeight):
        out = torch.empty((n, table.K), dtype=torch.float32, device=ids.device)
        check(lib().b200_get_rows_q(table.wtype, table.data.data_ptr(), table.K, table.M, ids.data_ptr(), out.data_ptr(),
                                    table.K * 4, n, _stream()))
        return out
    d = table.shape[1]
    out = torch.empty((n, d), dtype=torch.float32, device=ids.device)
    check(lib().b200_get_rows_f32(table.data_ptr(), table.stride(0) * 4, ids.data_ptr(), out.data_ptr(), d * 4, d, n, _stream()))
    return out


def argmax_rows(x: torch.Tensor) -> torch.Tensor:
    """First index of the maximum of every row of an f32 matrix (rows may be strided): the greedy choice the reference
    makes on the logits of a token (cactus/cactus_completion.cpp:210)."""
    assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    out = torch.empty(x.shape[0], dtype=torch.int32, device=x.device)
    check(lib().b200_argmax_rows(x.data_ptr(), x.stride(0) * 4, x.shape[1], x.shape[0], out.data_ptr(), _stream()))
    return out

"""Row-split mul_mat over the GPUs of one node: host side.

What a split buffer type does in the reference (lm_ggml_backend_split_buffer_type, cactus/ggml-backend.h:188,
requested for LLAMA_SPLIT_MODE_ROW at cactus/llama-model.cpp:339-351): rank r of g holds rows
[bounds[r], bounds[r+1]) of every mul_mat weight, computes that slice of the product, and the slices are joined so
that every rank continues with the whole activation (all other ops are replicated).  One process drives one GPU.
The join is ``b200_allgather_rows``: stores into every rank's output buffer through CUDA-IPC mapped peer memory and
a bounded flag wait; ``torch.distributed`` is used once, to pass the IPC handles around.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from ._lib import B200Error, check, lib


def row_bounds(M: int, g: int, tile: int = 16) -> list[int]:
    """Equal split of M rows over g ranks on ``tile``-row boundaries (the last rank takes the ragged tail)."""
    n_tiles = (M + tile - 1) // tile
    if n_tiles % g != 0:
        raise B200Error(f"{M} rows = {n_tiles} tiles of {tile} do not split evenly over {g} ranks")
    per = n_tiles // g
    return [min(M, r * per * tile) for r in range(g)] + [M]


def slice_blocks(blocks: np.ndarray, M: int, rank: int, g: int) -> np.ndarray:
    """Rows of ``rank`` out of a reference block stream [M, K/32*block_bytes] (rows are self-contained)."""
    b = row_bounds(M, g)
    return np.ascontiguousarray(blocks.reshape(M, -1)[b[rank]:b[rank + 1]])


class _Raw:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class RowSplit:
    """The shared output region of one rank and the mapped regions of its peers."""

    def __init__(self, rank: int, world: int, region_bytes: int, group=None):
        if not (1 <= world <= 8):
            raise B200Error("row split spans the GPUs of one node: at most 8 ranks")
        self.rank, self.world, self.region_bytes = rank, world, int(region_bytes)
        L = lib()
        self._own = []
        handles = []
        for nbytes in (self.region_bytes, 64):
            ptr, h = C.c_void_p(), C.create_string_buffer(64)
            check(L.b200_peer_alloc(nbytes, C.byref(ptr), h))
            self._own.append(ptr.value)
            handles.append(h.raw)
        everyone = [None] * world
        if world > 1:
            dist.all_gather_object(everyone, handles, group=group)
        else:
            everyone[0] = handles
        self._opened = []
        self.regions, self.flags = [], []
        for r in range(world):
            if r == rank:
                self.regions.append(self._own[0])
                self.flags.append(self._own[1])
                continue
            ptrs = []
            for h in everyone[r]:
                p = C.c_void_p()
                check(L.b200_peer_open(h, C.byref(p)))
                self._opened.append(p.value)
                ptrs.append(p.value)
            self.regions.append(ptrs[0])
            self.flags.append(ptrs[1])
        self._flag_arr = (C.c_void_p * world)(*self.flags)
        self._used = 0
        self._dst_arrays = {}

    def carve(self, *shape: int) -> torch.Tensor:
        """An f32 tensor in this rank's shared region; every rank must carve the same shapes in the same order."""
        n = int(np.prod(shape)) * 4
        off = (self._used + 255) // 256 * 256
        if off + n > self.region_bytes:
            raise B200Error("shared region too small")
        self._used = off + n
        t = torch.as_tensor(_Raw(self.regions[self.rank] + off, n), device="cuda").view(torch.float32).view(*shape)
        self._dst_arrays[t.data_ptr()] = (C.c_void_p * self.world)(*[base + off for base in self.regions])
        return t

    def allgather(self, src: torch.Tensor, T: int, Mg: int, dst: torch.Tensor, stream: int) -> None:
        """dst[:T, rank*Mg:(rank+1)*Mg] = src[:T, :Mg] on every rank; returns (in stream order) when all slices are in."""
        arr = self._dst_arrays[dst.data_ptr()]
        check(lib().b200_allgather_rows(src.data_ptr(), src.stride(0) * 4, T, Mg, self.rank, self.world, arr, dst.stride(0) * 4,
                                        self._flag_arr, stream))

    def mul_mat(self, w, act: torch.Tensor, T: int, dst: torch.Tensor, workspace: torch.Tensor, stream: int) -> None:
        """dst[:T, w.row0 : w.row0 + w.M] = this rank's rows of the product, stored by the mul_mat kernel's own write-back
        into every rank's dst; returns (in stream order) when all ranks' slices are in."""
        arr = self._dst_arrays[dst.data_ptr()]
        if w.parts is not None:   # this rank's rows of several tensors stacked: each piece has its own place in dst
            n = len(w.parts)
            rows = (C.c_int64 * n)(*[r for r, _ in w.parts])
            cols = (C.c_int64 * n)(*[c for _, c in w.parts])
            check(lib().b200_mul_mat_q_rowsplit_stacked(w.wtype, w.data.data_ptr(), w.K, w.M, act.data_ptr(), T, self.rank, self.world, arr,
                                                        dst.stride(0) * 4, n, rows, cols, workspace.data_ptr(), workspace.numel(), self._flag_arr, stream))
            return
        check(lib().b200_mul_mat_q_rowsplit(w.wtype, w.data.data_ptr(), w.K, w.M, act.data_ptr(), T, self.rank, self.world, arr, dst.stride(0) * 4,
                                            w.row0, workspace.data_ptr(), workspace.numel(), self._flag_arr, stream))

    def status(self) -> int:
        """0, or 1 + the first rank whose slice did not arrive within the wait limit."""
        return int(lib().b200_peer_status(self.flags[self.rank]))

    def close(self) -> None:
        L = lib()
        torch.cuda.synchronize()
        if self.world > 1 and dist.is_initialized():
            dist.barrier()   # nobody unmaps while a peer may still push
        for p in self._opened:
            L.b200_peer_close(p)
        self._opened = []
        if self.world > 1 and dist.is_initialized():
            dist.barrier()
        for p in self._own:
            L.b200_peer_free(p)
        self._own = []

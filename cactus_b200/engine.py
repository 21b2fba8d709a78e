"""A llama decode step as the ggml graph of the reference lays it out, issued through the C ABI.

Node order and shapes follow llm_build_llama (cactus/llama-model.cpp:4517-4671) with flash attention on
and the unified f16 KV cache of llama_kv_cache_unified (cactus/llama-kv-cache.cpp:25-138): per layer
RMS_NORM*w -> wq/wk/wv MUL_MAT -> ROPE(q, k) -> K/V store -> FLASH_ATTN_EXT -> wo MUL_MAT -> ADD ->
RMS_NORM*w -> gate/up MUL_MAT -> SILU*up -> down MUL_MAT -> ADD; then the final norm and the output head.

torch is used for device memory, the stream and CUDA-graph capture only; every node is a call into
libcactus_b200.so.  This is the host driver the benchmark and the model-level tests use; inside cactus the
same calls are issued by the ggml backend plug-in from graph_compute.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np
import torch

from ._lib import check, lib
from .ops import Q4_0, Q8_0, Q8_AVX2, QWeight


@dataclass
class LlamaConfig:
    n_layer: int
    d_model: int
    n_head: int
    n_kv_head: int
    d_ff: int
    vocab: int
    rope_theta: float = 500000.0
    eps: float = 1e-5
    layer_type: int = Q4_0      # quantisation of the layer weights
    head_type: int = Q4_0       # quantisation of token_embd / output

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_head

    def mul_mat_shapes(self):
        """(name, K, M) of the seven MUL_MATs of a layer (cactus/llama-model.cpp:1745-1771)."""
        d, kv, ff = self.d_model, self.n_kv_head * self.head_dim, self.d_ff
        return [("wq", d, d), ("wk", d, kv), ("wv", d, kv), ("wo", d, d), ("gate", d, ff), ("up", d, ff), ("down", ff, d)]

    def weight_bytes_per_step(self) -> int:
        """Bytes of quantised weights one decode step streams (the mul_mat term of the HBM roofline)."""
        bb = {Q4_0: 18, Q8_0: 34}
        per_layer = sum(M * (K // 32) * bb[self.layer_type] for _, K, M in self.mul_mat_shapes())
        return self.n_layer * per_layer + self.vocab * (self.d_model // 32) * bb[self.head_type]


LLAMA_3_8B = LlamaConfig(32, 4096, 32, 8, 14336, 128256)
LLAMA_32_1B = LlamaConfig(16, 2048, 32, 8, 8192, 128256, head_type=Q8_0)
LLAMA_3_70B = LlamaConfig(80, 8192, 64, 8, 28672, 128256)


def random_blocks(wtype: int, M: int, K: int, gen: torch.Generator, std: float = 0.02, rows_per_chunk: int = 8192) -> torch.Tensor:
    """Random N(0, std) weights quantised on the device into the reference's row-major block stream
    (quantize_row_q4_0_ref / quantize_row_q8_0_ref arithmetic, cactus/ggml-quants.c:25-60, 188-211).
    Synthetic-data plumbing for benchmarks; parity tests quantise with the oracle instead."""
    nb = K // 32
    bb = 18 if wtype == Q4_0 else 34
    out = torch.empty((M, nb, bb), dtype=torch.uint8, device="cuda")
    for r0 in range(0, M, rows_per_chunk):
        r1 = min(M, r0 + rows_per_chunk)
        x = (torch.randn((r1 - r0, nb, 32), device="cuda", generator=gen) * std)
        if wtype == Q4_0:
            idx = x.abs().argmax(dim=-1, keepdim=True)
            mx = x.gather(-1, idx)
            d = mx / -8.0
            inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
            q = torch.clamp(torch.trunc(x * inv + 8.5), max=15).to(torch.uint8)
            out[r0:r1, :, 2:] = q[..., :16] | (q[..., 16:] << 4)
        else:
            d = x.abs().amax(dim=-1, keepdim=True) / 127.0
            inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
            v = x * inv
            q = (torch.sign(v) * torch.floor(v.abs() + 0.5)).to(torch.int8)
            out[r0:r1, :, 2:] = q.view(torch.uint8)
        out[r0:r1, :, :2] = d.to(torch.float16).view(torch.uint8).reshape(r1 - r0, nb, 2)
    return out.reshape(M, nb * bb)


class LlamaWeights:
    """Device-resident weights in the tiled layout.  ``tensors`` maps ggml tensor names to QWeight / f32 tensors."""

    def __init__(self, cfg: LlamaConfig):
        self.cfg = cfg
        self.tensors: dict[str, object] = {}

    @staticmethod
    def random(cfg: LlamaConfig, seed: int = 0, rank: int = 0, world: int = 1) -> "LlamaWeights":
        """Synthetic weights.  With ``world`` > 1 only this rank's rows of the mul_mat weights are generated (row
        split); the embedding table, which every rank reads whole, comes from the shared seed."""
        w = LlamaWeights(cfg)
        gen = torch.Generator(device="cuda").manual_seed(seed)
        d = cfg.d_model
        w.tensors["token_embd.weight"] = QWeight.from_blocks(cfg.head_type, d, cfg.vocab, random_blocks(cfg.head_type, cfg.vocab, d, gen))
        if world > 1:
            from .rowsplit import row_bounds
            gen = torch.Generator(device="cuda").manual_seed(seed * 1000 + 17 + rank)
        rows = (lambda M: M) if world == 1 else (lambda M: row_bounds(M, world)[rank + 1] - row_bounds(M, world)[rank])
        row0 = (lambda M: 0) if world == 1 else (lambda M: row_bounds(M, world)[rank])

        def make(wtype, K, M):
            q = QWeight.from_blocks(wtype, K, rows(M), random_blocks(wtype, rows(M), K, gen))
            q.row0 = row0(M)
            return q
        w.tensors["output.weight"] = make(cfg.head_type, d, cfg.vocab)
        w.tensors["output_norm.weight"] = torch.ones(d, device="cuda")
        names = {"wq": "attn_q", "wk": "attn_k", "wv": "attn_v", "wo": "attn_output", "gate": "ffn_gate", "up": "ffn_up", "down": "ffn_down"}
        for il in range(cfg.n_layer):
            for short, K, M in cfg.mul_mat_shapes():
                w.tensors[f"blk.{il}.{names[short]}.weight"] = make(cfg.layer_type, K, M)
            w.tensors[f"blk.{il}.attn_norm.weight"] = torch.ones(d, device="cuda")
            w.tensors[f"blk.{il}.ffn_norm.weight"] = torch.ones(d, device="cuda")
        return w

    def shard(self, rank: int, g: int) -> "LlamaWeights":
        """This rank's rows of every mul_mat weight (attention, feed-forward, output head); the embedding table and
        the norm weights stay whole, as the replicated ops need them."""
        from .rowsplit import row_bounds
        out = LlamaWeights(self.cfg)
        for name, t in self.tensors.items():
            if isinstance(t, QWeight) and name != "token_embd.weight":
                b = row_bounds(t.M, g)
                out.tensors[name] = t.row_slice(b[rank], b[rank + 1])
            else:
                out.tensors[name] = t
        return out

    @staticmethod
    def from_numpy(cfg: LlamaConfig, arrays: dict) -> "LlamaWeights":
        """arrays: name -> uint8 block stream [M, K/32*bb] for quantised tensors, f32 [d] for norms."""
        w = LlamaWeights(cfg)
        d = cfg.d_model
        kinds = {"attn_q": "wq", "attn_k": "wk", "attn_v": "wv", "attn_output": "wo", "ffn_gate": "gate", "ffn_up": "up", "ffn_down": "down"}
        dims = {s: (K, M) for s, K, M in cfg.mul_mat_shapes()}
        for name, a in arrays.items():
            if name.endswith("norm.weight"):
                w.tensors[name] = torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()
            elif name in ("token_embd.weight", "output.weight"):
                w.tensors[name] = QWeight.from_blocks(cfg.head_type, d, cfg.vocab, a)
            else:
                K, M = dims[kinds[name.split(".")[2]]]
                w.tensors[name] = QWeight.from_blocks(cfg.layer_type, K, M, a)
        return w


class LlamaEngine:
    """Runs ubatches (ragged sets of tokens from many sequences) through the model.

    ``decode(tokens, pos, seq, slots)`` mirrors what llama_context::decode (cactus/llama-context.cpp:849-1143)
    does for one ubatch after find_slot has chosen the cache cells: host int32 arrays in, host f32 logits
    [n_tokens, vocab] out.  The device-side work for a given token count is captured once as a CUDA graph
    (all kernel arguments are static: cells are addressed through the ``slots`` array and the attention
    always spans the whole cache, masked) and replayed for every later ubatch of that size.
    """

    def __init__(self, weights: LlamaWeights, n_cells: int, max_tokens: int = 512, variant: int = Q8_AVX2, use_graphs: bool = True, split=None,
                 fuse_weights: bool = True, head_parallel: bool = True):
        assert n_cells % 256 == 0, "the cache is padded to 256 cells for flash attention (cactus/llama-kv-cache.cpp:20-23)"
        self.w, self.cfg, self.n_cells, self.max_tokens, self.variant = weights, weights.cfg, n_cells, max_tokens, variant
        self.use_graphs = use_graphs
        # up to this many tokens the attention leaves its output quantised itself (b200_flash_attn_ext_quant: one launch
        # less per layer, bit-identical).  Off: measured on B200 it is slower at every token count -- one sequence of the
        # 8B architecture 2.52-2.58 ms per token against 2.40 with the separate quantiser, the 64-token batch 70.5 us per
        # attention against 57.5 + 2.5 (the attention kernel sits at its register limit).  B200_FA_QUANT_MAX_T sets it.
        self.fa_quant_max_tokens = int(os.environ.get("B200_FA_QUANT_MAX_T", "0"))
        # row split (cactus_b200.rowsplit.RowSplit): ``weights`` then holds this rank's rows of every mul_mat weight,
        # each product is joined into buffers the peers can write, everything else is replicated
        self.split = split
        g = split.world if split is not None else 1
        cfg, L = self.cfg, lib()
        # wq/wk/wv and gate/up read the same activations: stacked into one weight each, they are one mul_mat each (the
        # engine takes the stacked copies and drops the separate tensors).
        # With a row split the rank's slices are stacked the same way; each piece then carries the column of the joined
        # output where its rows belong (QWeight.parts), and one product stores all of them.
        self.fused = bool(fuse_weights)
        # Row split with the heads of a rank kept at home: wq/wk/wv cut by rows are cut by heads, so a rank rotates, caches
        # and attends its own H/g query and Hkv/g KV heads only (its share of the cache, too) and the ranks exchange the
        # attention output instead of q, k and v: attention time and cache memory divide by g.
        self.hp = bool(head_parallel) and split is not None and self.fused and cfg.n_head % g == 0 and cfg.n_kv_head % g == 0 and \
            (cfg.n_kv_head // g * cfg.head_dim) % 16 == 0
        if self.fused:
            t = self.w.tensors
            kvd_ = cfg.n_kv_head * cfg.head_dim

            def stack(ws, bases):
                out = QWeight.cat(ws)
                if split is not None:
                    out.parts = [(w_.M, base + w_.row0) for w_, base in zip(ws, bases)]
                return out
            for il in range(cfg.n_layer):
                p = f"blk.{il}."
                if p + "attn_qkv.weight" not in t:
                    t[p + "attn_qkv.weight"] = stack([t.pop(p + "attn_q.weight"), t.pop(p + "attn_k.weight"), t.pop(p + "attn_v.weight")],
                                                     [0, cfg.d_model, cfg.d_model + kvd_])
                    if self.hp:
                        t[p + "attn_qkv.weight"].parts = None   # the product stays on this rank
                    t[p + "ffn_gate_up.weight"] = stack([t.pop(p + "ffn_gate.weight"), t.pop(p + "ffn_up.weight")], [0, cfg.d_ff])
        dev = "cuda"
        self.n_head_local = cfg.n_head // g if self.hp else cfg.n_head
        self.n_kv_head_local = cfg.n_kv_head // g if self.hp else cfg.n_kv_head
        kvd = self.n_kv_head_local * cfg.head_dim      # K/V row of one cell as this rank caches it
        qd = self.n_head_local * cfg.head_dim          # q row of one token as this rank holds it
        T = max_tokens
        f32 = lambda *s: torch.empty(s, dtype=torch.float32, device=dev)  # noqa: E731
        u8 = lambda n: torch.empty(max(int(n), 256), dtype=torch.uint8, device=dev)  # noqa: E731
        self.k_cache = [torch.zeros((n_cells, kvd), dtype=torch.float16, device=dev) for _ in range(cfg.n_layer)]
        self.v_cache = [torch.zeros((n_cells, kvd), dtype=torch.float16, device=dev) for _ in range(cfg.n_layer)]
        self.cell_pos = torch.full((n_cells,), -1, dtype=torch.int32, device=dev)
        self.cell_seq = torch.full((n_cells,), -1, dtype=torch.int32, device=dev)
        # per-ubatch inputs: rows = tokens, pos, seq, slots
        self.inp = torch.zeros((4, T), dtype=torch.int32, device=dev)
        self.inp_host = torch.zeros((4, T), dtype=torch.int32).pin_memory()
        self.mask = torch.empty(((T + 63) // 64 * 64, n_cells), dtype=torch.float16, device=dev)
        self.index = u8(L.b200_mask_index_bytes(T, n_cells))
        self.x, self.h, self.attn = f32(T, cfg.d_model), f32(T, cfg.d_model), f32(T, cfg.d_model)
        out = split.carve if split is not None else f32   # mul_mat outputs: where the peers' slices land
        if self.fused:   # the stacked products, and the reference's q/k/v and gate/up as column ranges of them
            self.qkv, self.gu = (f32 if self.hp else out)(T, qd + 2 * kvd), out(T, 2 * cfg.d_ff)
            self.q, self.k, self.v = self.qkv[:, :qd], self.qkv[:, qd:qd + kvd], self.qkv[:, qd + kvd:]
            if self.hp:   # this rank's heads of the attention output, and the joined output every rank continues with
                self.attn_part, self.attn = f32(T, qd), out(T, cfg.d_model)
            self.gate, self.up = self.gu[:, :cfg.d_ff], self.gu[:, cfg.d_ff:]
        else:
            self.q, self.k, self.v = out(T, cfg.d_model), out(T, kvd), out(T, kvd)
            self.gate, self.up = out(T, cfg.d_ff), out(T, cfg.d_ff)
        self.tmp, self.tmp2 = out(T, cfg.d_model), out(T, cfg.d_model)   # attention branch / feed-forward branch of the residual
        self.logits = out(T, cfg.vocab)
        self.next_ids = torch.zeros(T, dtype=torch.int32, device=dev)
        self.logits_host = torch.empty((T, cfg.vocab), dtype=torch.float32).pin_memory()
        self.ids_host = torch.zeros(T, dtype=torch.int32).pin_memory()
        self.act_d = u8(L.b200_act_bytes(cfg.d_model, T))
        self.act_ff = u8(L.b200_act_bytes(cfg.d_ff, T))
        kvd_all = cfg.n_kv_head * cfg.head_dim
        shapes = [(K, M // g) for _, K, M in cfg.mul_mat_shapes()] + [(cfg.d_model, (cfg.d_model + 2 * kvd_all) // g), (cfg.d_model, 2 * cfg.d_ff // g)]
        ws = [L.b200_mul_mat_workspace_bytes(cfg.layer_type, K, M, t) for K, M in shapes for t in range(1, T + 1)]
        ws += [L.b200_mul_mat_workspace_bytes(cfg.head_type, cfg.d_model, cfg.vocab // g, t) for t in range(1, T + 1)]
        self.ws = u8(max(ws))
        self.fa_scratch = u8(max(L.b200_flash_attn_scratch_bytes(cfg.head_dim, self.n_head_local, self.n_kv_head_local, t, n_cells) for t in range(1, T + 1)))
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.launches_per_step: dict[int, int] = {}

    # ---- one ubatch worth of kernels on the current stream -------------------------------------
    def _mm(self, name: str, act: torch.Tensor, T: int, out: torch.Tensor):
        w: QWeight = self.w.tensors[name]
        if self.split is None:
            check(lib().b200_mul_mat_q_prequant(w.wtype, w.data.data_ptr(), w.K, w.M, act.data_ptr(), T, out.data_ptr(), out.stride(0) * 4,
                                                self.ws.data_ptr(), self.ws.numel(), self._st))
            return
        if self.hp and name.endswith("attn_qkv.weight"):   # q, k, v of this rank's heads: nobody else needs them
            check(lib().b200_mul_mat_q_prequant(w.wtype, w.data.data_ptr(), w.K, w.M, act.data_ptr(), T, out.data_ptr(), out.stride(0) * 4,
                                                self.ws.data_ptr(), self.ws.numel(), self._st))
            return
        self.split.mul_mat(w, act, T, out, self.ws, self._st)   # this rank's rows, written into every rank's `out`, then the flag exchange

    def _quant(self, x: torch.Tensor, K: int, T: int, act: torch.Tensor):
        check(lib().b200_quantize_activations(x.data_ptr(), x.stride(0) * 4, K, T, act.data_ptr(), act.numel(), self.variant, self._st))

    def enqueue(self, T: int) -> None:
        cfg, L = self.cfg, lib()
        st = self._st = torch.cuda.current_stream().cuda_stream
        D, H, Hkv, d, nkv = cfg.head_dim, self.n_head_local, self.n_kv_head_local, cfg.d_model, self.n_cells
        kvd = Hkv * D
        tokens, pos, seq, slots = (self.inp[i].data_ptr() for i in range(4))
        # cell bookkeeping, mask and its index (shared by all layers)
        check(L.b200_scatter_i32(self.cell_pos.data_ptr(), slots, pos, T, st))
        check(L.b200_scatter_i32(self.cell_seq.data_ptr(), slots, seq, T, st))
        check(L.b200_kq_mask_build(self.cell_pos.data_ptr(), self.cell_seq.data_ptr(), nkv, pos, seq, T, self.mask.data_ptr(), nkv * 2, st))
        check(L.b200_mask_index_build(self.mask.data_ptr(), nkv * 2, T, nkv, self.index.data_ptr(), self.index.numel(), st))
        emb: QWeight = self.w.tensors["token_embd.weight"]
        check(L.b200_get_rows_q(emb.wtype, emb.data.data_ptr(), emb.K, emb.M, tokens, self.x.data_ptr(), d * 4, T, st))
        x = self.x
        V = self.variant

        def norm_quant(weight: str, residual):
            """x (+= residual) -> rms_norm * weight -> quantised into act_d; one launch"""
            check(L.b200_add_rms_norm_quantize(x.data_ptr(), d * 4, residual.data_ptr() if residual is not None else None, d * 4,
                                               self.w.tensors[weight].data_ptr(), None, 0, d, T, cfg.eps, self.act_d.data_ptr(), self.act_d.numel(), V, st))

        pending = None   # the residual branch not yet added to x: folded into the next norm
        for il in range(cfg.n_layer):
            p = f"blk.{il}."
            norm_quant(p + "attn_norm.weight", pending)
            if self.fused:
                self._mm(p + "attn_qkv.weight", self.act_d, T, self.qkv)
            else:
                self._mm(p + "attn_q.weight", self.act_d, T, self.q)
                self._mm(p + "attn_k.weight", self.act_d, T, self.k)
                self._mm(p + "attn_v.weight", self.act_d, T, self.v)
            kc, vc = self.k_cache[il], self.v_cache[il]
            qs, kst, vst = self.q.stride(0) * 4, self.k.stride(0) * 4, self.v.stride(0) * 4
            check(L.b200_rope_store(self.q.data_ptr(), D * 4, qs, self.k.data_ptr(), D * 4, kst, self.v.data_ptr(), vst, D, H, Hkv, T, D,
                                    pos, None, cfg.rope_theta, 1.0, 1.0, slots, kc.data_ptr(), kvd * 2, vc.data_ptr(), kvd * 2, st))
            attn_args = (D, H, Hkv, T, nkv, self.q.data_ptr(), qs, D * 4, kc.data_ptr(), kvd * 2, D * 2, vc.data_ptr(), kvd * 2, D * 2,
                         self.mask.data_ptr(), nkv * 2, self.index.data_ptr(), D ** -0.5, 0.0, 0.0)
            if T <= self.fa_quant_max_tokens and not self.hp:
                check(L.b200_flash_attn_ext_quant(*attn_args, None, self.act_d.data_ptr(), self.act_d.numel(), V, self.fa_scratch.data_ptr(),
                                                  self.fa_scratch.numel(), st))
            else:
                check(L.b200_flash_attn_ext_indexed(*attn_args, (self.attn_part if self.hp else self.attn).data_ptr(), self.fa_scratch.data_ptr(),
                                                    self.fa_scratch.numel(), st))
                if self.hp:   # every rank's heads side by side, on every rank
                    self.split.allgather(self.attn_part, T, H * D, self.attn, st)
                self._quant(self.attn, d, T, self.act_d)
            self._mm(p + "attn_output.weight", self.act_d, T, self.tmp)
            norm_quant(p + "ffn_norm.weight", self.tmp)
            if self.fused:
                self._mm(p + "ffn_gate_up.weight", self.act_d, T, self.gu)
            else:
                self._mm(p + "ffn_gate.weight", self.act_d, T, self.gate)
                self._mm(p + "ffn_up.weight", self.act_d, T, self.up)
            check(L.b200_silu_mul_quantize(self.gate.data_ptr(), self.up.data_ptr(), self.gate.stride(0) * 4, None, 0, cfg.d_ff, T, self.act_ff.data_ptr(),
                                           self.act_ff.numel(), V, st))
            self._mm(p + "ffn_down.weight", self.act_ff, T, self.tmp2)
            pending = self.tmp2
        check(L.b200_add_rms_norm_quantize(x.data_ptr(), d * 4, pending.data_ptr(), d * 4, self.w.tensors["output_norm.weight"].data_ptr(), None, 0,
                                           d, T, cfg.eps, self.act_d.data_ptr(), self.act_d.numel(), V, st))
        self._mm("output.weight", self.act_d, T, self.logits)
        check(L.b200_argmax_rows(self.logits.data_ptr(), cfg.vocab * 4, cfg.vocab, T, self.next_ids.data_ptr(), st))

    def run_device(self, T: int) -> None:
        """Runs one ubatch of T tokens whose inputs are already in ``self.inp`` (device)."""
        if not self.use_graphs:
            self.enqueue(T)
            return
        g = self.graphs.get(T)
        if g is None:
            L = lib()
            # warm up outside capture (first-use attribute settings), on a side stream as capture requires
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            saved = (self.cell_pos.clone(), self.cell_seq.clone())
            with torch.cuda.stream(s):
                self.enqueue(T)
                before = L.b200_launch_count()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=s):
                    self.enqueue(T)
                self.launches_per_step[T] = int(L.b200_launch_count() - before)
            torch.cuda.current_stream().wait_stream(s)
            self.cell_pos.copy_(saved[0])
            self.cell_seq.copy_(saved[1])
            self.graphs[T] = g
        g.replay()

    def decode(self, tokens, pos, seq, slots, want_logits: bool = True):
        """Host arrays in, host logits [T, vocab] (and greedy next ids [T]) out.  Blocks until done."""
        T = len(tokens)
        assert 0 < T <= self.max_tokens
        ih = self.inp_host
        ih[0, :T] = torch.as_tensor(np.asarray(tokens, np.int32))
        ih[1, :T] = torch.as_tensor(np.asarray(pos, np.int32))
        ih[2, :T] = torch.as_tensor(np.asarray(seq, np.int32))
        ih[3, :T] = torch.as_tensor(np.asarray(slots, np.int32))
        self.inp.copy_(ih, non_blocking=True)
        self.run_device(T)
        if want_logits:
            self.logits_host[:T].copy_(self.logits[:T], non_blocking=True)
        self.ids_host[:T].copy_(self.next_ids[:T], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        if self.split is not None:
            # a join whose bounded wait ran out leaves a peer's rows stale in the joined buffers: the logits are not to be trusted
            st = self.split.status()
            if st != 0:
                from ._lib import B200Error
                raise B200Error(f"row split: the rows of rank {st - 1} did not arrive within the wait limit")
        return (self.logits_host[:T].numpy() if want_logits else None), self.ids_host[:T].numpy()

    def clear(self):
        self.cell_pos.fill_(-1)
        self.cell_seq.fill_(-1)

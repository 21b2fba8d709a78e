"""Small single-kernel workloads for timing and profiling (run under ncu on a GPU box):

    python -m cactus_b200.microbench mul_mat --K 4096 --M 14336 --N 64 --copies 8 --reps 3
    python -m cactus_b200.microbench fattn --seqs 64 --ctx 900 --reps 3
    python -m cactus_b200.microbench fattn --cfg2 a --copies 8       # the 512-token prefill ubatch of 16 ragged sequences
    python -m cactus_b200.microbench quantize --K 4096 --N 64
    python -m cactus_b200.microbench decode --seqs 1 --ctx 2048 --layers 32   # whole decode steps of the 8B architecture
    python -m cactus_b200.microbench umma-rate                      # tcgen05.mma issue rates per kind and shape (csrc/probes)

`--copies` distinct weight tensors are cycled so the weights streamed per pass exceed the 126 MB L2.
Prints one JSON line with the CUDA-event time per launch and the algorithmic GB/s.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

from . import ops
from ._lib import check, lib
from .engine import random_blocks


def time_launches(fn, reps):
    best = None
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        n = fn()
        e1.record()
        e1.synchronize()
        ms = e0.elapsed_time(e1) / n
        best = ms if best is None else min(best, ms)
    return best


def bench_mul_mat(a):
    L = lib()
    gen = torch.Generator(device="cuda").manual_seed(0)
    ws = [ops.QWeight.from_blocks(a.wtype, a.K, a.M, random_blocks(a.wtype, a.M, a.K, gen)) for _ in range(a.copies)]
    x = torch.randn((a.N, a.K), device="cuda", generator=gen)
    out = torch.empty((a.N, a.M), device="cuda")
    act = torch.empty(L.b200_act_bytes(a.K, a.N), dtype=torch.uint8, device="cuda")
    wsp = torch.empty(max(256, L.b200_mul_mat_workspace_bytes(a.wtype, a.K, a.M, a.N)), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    check(L.b200_quantize_activations(x.data_ptr(), a.K * 4, a.K, a.N, act.data_ptr(), act.numel(), 0, st))

    def run():
        st = torch.cuda.current_stream().cuda_stream   # the capture stream while a graph is being recorded
        for w in ws:
            check(L.b200_mul_mat_q_prequant(w.wtype, w.data.data_ptr(), w.K, w.M, act.data_ptr(), a.N, out.data_ptr(), a.M * 4,
                                            wsp.data_ptr(), wsp.numel(), st))
        return len(ws)

    run()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    ms = time_launches(lambda: (g.replay(), len(ws))[1], a.reps)
    bb = 18 if a.wtype == 2 else 34
    alg = a.M * (a.K // 32) * bb + a.N * a.K * 4 + a.N * a.M * 4
    return {"kernel": "mul_mat", "K": a.K, "M": a.M, "N": a.N, "wtype": a.wtype, "ms_per_launch": ms, "GBps": alg / ms / 1e6,
            "TOPS": 2 * a.M * a.N * a.K / ms / 1e9}


def bench_fattn(a):
    L = lib()
    gen = torch.Generator(device="cuda").manual_seed(0)
    D, H, Hkv = a.D, a.H, a.Hkv
    if a.ragged:   # the benchmark's 64 prompt lengths (U[16, 2048] scaled to the 65536-cell cache), contiguous runs per sequence
        from .workloads import prompt_lengths
        lens = torch.from_numpy(prompt_lengths()[0]).to("cuda")
        a.seqs = int(lens.numel())
    else:
        lens = torch.full((a.seqs,), a.ctx, dtype=torch.int64, device="cuda")
    total = int(lens.sum())
    n_cells = (total + 255) // 256 * 256
    layers = a.copies
    ks = [torch.randn((n_cells, Hkv * D), device="cuda", generator=gen).half() for _ in range(layers)]
    vs = [torch.randn((n_cells, Hkv * D), device="cuda", generator=gen).half() for _ in range(layers)]
    # --head-major: the same bytes addressed as [Hkv][cells][D] (a layout experiment: the reference's cache is cell-major)
    nb_cell, nb_head = (D * 2, n_cells * D * 2) if a.head_major else (Hkv * D * 2, D * 2)
    q = torch.randn((a.seqs, H * D), device="cuda", generator=gen)
    ends = torch.cumsum(lens, 0)
    cells = torch.arange(n_cells, device="cuda")
    owner = torch.searchsorted(ends, cells, right=True)
    cell_seq = owner.to(torch.int32)
    cell_seq[cells >= total] = -1
    starts = ends - lens
    cell_pos = (cells - starts[owner.clamp(max=a.seqs - 1)]).to(torch.int32)
    tok_pos = (lens - 1).to(torch.int32)
    tok_seq = torch.arange(a.seqs, dtype=torch.int32, device="cuda")
    mask = torch.empty(((a.seqs + 63) // 64 * 64, n_cells), dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    check(L.b200_kq_mask_build(cell_pos.data_ptr(), cell_seq.data_ptr(), n_cells, tok_pos.data_ptr(), tok_seq.data_ptr(), a.seqs,
                               mask.data_ptr(), n_cells * 2, st))
    index = torch.empty(L.b200_mask_index_bytes(a.seqs, n_cells), dtype=torch.uint8, device="cuda")
    check(L.b200_mask_index_build(mask.data_ptr(), n_cells * 2, a.seqs, n_cells, index.data_ptr(), index.numel(), st))
    scratch = torch.empty(max(256, L.b200_flash_attn_scratch_bytes(D, H, Hkv, a.seqs, n_cells)), dtype=torch.uint8, device="cuda")
    out = torch.empty((a.seqs, H * D), device="cuda")
    act = torch.empty(L.b200_act_bytes(H * D, a.seqs), dtype=torch.uint8, device="cuda")

    def run():
        st = torch.cuda.current_stream().cuda_stream
        for k, v in zip(ks, vs):
            if a.quant:   # the output left as the quantised activations of the next mul_mat only
                check(L.b200_flash_attn_ext_quant(D, H, Hkv, a.seqs, n_cells, q.data_ptr(), H * D * 4, D * 4, k.data_ptr(), nb_cell, nb_head,
                                                  v.data_ptr(), nb_cell, nb_head, mask.data_ptr(), n_cells * 2, index.data_ptr(),
                                                  D ** -0.5, 0.0, 0.0, None, act.data_ptr(), act.numel(), 0, scratch.data_ptr(), scratch.numel(), st))
                continue
            check(L.b200_flash_attn_ext_indexed(D, H, Hkv, a.seqs, n_cells, q.data_ptr(), H * D * 4, D * 4, k.data_ptr(), nb_cell, nb_head,
                                                v.data_ptr(), nb_cell, nb_head, mask.data_ptr(), n_cells * 2, index.data_ptr(),
                                                D ** -0.5, 0.0, 0.0, out.data_ptr(), scratch.data_ptr(), scratch.numel(), st))
        return layers

    run()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    ms = time_launches(lambda: (g.replay(), layers)[1], a.reps)
    alg = total * Hkv * D * 2 * 2 + 2 * a.seqs * H * D * 4
    return {"kernel": "flash_attn_ext", "seqs": a.seqs, "ctx": "ragged" if a.ragged else a.ctx, "cells": total, "D": D, "H": H, "Hkv": Hkv, "ms_per_launch": ms, "GBps": alg / ms / 1e6}


def bench_fattn_prefill(a):
    """The single FLASH_ATTN_EXT op of a prefill ubatch: 32 query heads / 8 KV heads, head 128, 16 sequences with
    contexts ~ U[64, 4096] and 1-256 query tokens each (seed 0), causal + per-slot sequence mask.
    variant a: contexts rescaled to fit 8192 slots, query tokens clipped to a 512-token ubatch;
    variant b: the cache enlarged to pad256(sum of contexts), lengths as drawn, still one ubatch of at most 512 tokens."""
    L = lib()
    D, H, Hkv = a.D, a.H, a.Hkv
    rng = np.random.default_rng(0)
    ctx = rng.integers(64, 4097, 16)
    nq = rng.integers(1, 257, 16)
    if a.cfg2 == "a":
        ctx = np.maximum(64, (ctx * min(1.0, 8192 / ctx.sum() * 0.999)).astype(int))
        while ctx.sum() > 8192:
            ctx[np.argmax(ctx)] -= ctx.sum() - 8192
    nq = np.minimum(nq, ctx)
    nq = np.maximum(1, (nq * min(1.0, 512 / nq.sum())).astype(int))
    total = int(ctx.sum())
    n_cells = (total + 255) // 256 * 256
    cell_pos = np.full(n_cells, -1, np.int32)
    cell_seq = np.full(n_cells, -1, np.int32)
    head = 0
    for s_, n in enumerate(ctx):
        cell_pos[head:head + n] = np.arange(n)
        cell_seq[head:head + n] = s_
        head += n
    tok_pos = np.concatenate([np.arange(c - q_, c) for c, q_ in zip(ctx, nq)]).astype(np.int32)
    tok_seq = np.concatenate([np.full(q_, s_) for s_, q_ in enumerate(nq)]).astype(np.int32)
    Nq = len(tok_pos)
    gen = torch.Generator(device="cuda").manual_seed(0)
    layers = a.copies
    ks = [torch.randn((n_cells, Hkv * D), device="cuda", generator=gen).half() for _ in range(layers)]
    vs = [torch.randn((n_cells, Hkv * D), device="cuda", generator=gen).half() for _ in range(layers)]
    q = torch.randn((Nq, H * D), device="cuda", generator=gen)
    mask = torch.empty(((Nq + 63) // 64 * 64, n_cells), dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    dv = lambda x: torch.from_numpy(x).cuda()  # noqa: E731
    cp, cs, tp, ts = dv(cell_pos), dv(cell_seq), dv(tok_pos), dv(tok_seq)
    check(L.b200_kq_mask_build(cp.data_ptr(), cs.data_ptr(), n_cells, tp.data_ptr(), ts.data_ptr(), Nq, mask.data_ptr(), n_cells * 2, st))
    index = torch.empty(L.b200_mask_index_bytes(Nq, n_cells), dtype=torch.uint8, device="cuda")
    check(L.b200_mask_index_build(mask.data_ptr(), n_cells * 2, Nq, n_cells, index.data_ptr(), index.numel(), st))
    scratch = torch.empty(max(256, L.b200_flash_attn_scratch_bytes(D, H, Hkv, Nq, n_cells)), dtype=torch.uint8, device="cuda")
    out = torch.empty((Nq, H * D), device="cuda")

    def run():
        st = torch.cuda.current_stream().cuda_stream
        for k, v in zip(ks, vs):
            check(L.b200_flash_attn_ext_indexed(D, H, Hkv, Nq, n_cells, q.data_ptr(), H * D * 4, D * 4, k.data_ptr(), Hkv * D * 2, D * 2,
                                                v.data_ptr(), Hkv * D * 2, D * 2, mask.data_ptr(), n_cells * 2, index.data_ptr(),
                                                D ** -0.5, 0.0, 0.0, out.data_ptr(), scratch.data_ptr(), scratch.numel(), st))
        return layers

    run()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    ms = time_launches(lambda: (g.replay(), layers)[1], a.reps)
    # algorithmic bytes: every sequence's attended K/V once per kv-head, Q in, O out, the f16 mask once
    alg = total * Hkv * D * 2 * 2 + 2 * Nq * H * D * 4 + n_cells * ((Nq + 63) // 64 * 64) * 2
    # flops: 2 * H * (DK + DV) per (query token, attended cell) pair
    pairs = int(sum(int(c) * int(q_) - int(q_) * (int(q_) - 1) // 2 for c, q_ in zip(ctx, nq)))
    flops = 2 * H * 2 * D * pairs
    return {"kernel": "flash_attn_ext prefill", "variant": a.cfg2, "tokens": Nq, "sequences": 16, "cells": total, "D": D, "H": H, "Hkv": Hkv,
            "ms_per_launch": ms, "TFLOPs": flops / ms / 1e9, "GBps": alg / ms / 1e6, "attended_pairs": pairs}


def bench_quantize(a):
    L = lib()
    x = torch.randn((a.N, a.K), device="cuda")
    act = torch.empty(L.b200_act_bytes(a.K, a.N), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream

    def run():
        for _ in range(20):
            check(L.b200_quantize_activations(x.data_ptr(), a.K * 4, a.K, a.N, act.data_ptr(), act.numel(), 0, st))
        return 20

    run()
    ms = time_launches(run, a.reps)
    return {"kernel": "quantize_q8_0", "K": a.K, "N": a.N, "ms_per_launch": ms, "GBps": (a.N * a.K * 4 + a.N * a.K * 34 / 32) / ms / 1e6}


def bench_decode(a):
    """Whole decode steps of the Llama-3-8B architecture (`--layers` of its layers) on the graph engine: `--seqs` sequences
    of `--ctx` cached cells each, one token per sequence and step, inputs resident on the device."""
    from dataclasses import replace

    from .engine import LLAMA_3_8B, LlamaEngine, LlamaWeights
    cfg = replace(LLAMA_3_8B, n_layer=a.layers)
    S, ctx = a.seqs, a.ctx
    steps = 16
    n_cells = max(a.cells, (S * (ctx + steps + 4) + 255) // 256 * 256)
    eng = LlamaEngine(LlamaWeights.random(cfg, seed=0), n_cells, max_tokens=S)
    gen = torch.Generator(device="cuda").manual_seed(1)
    for il in range(cfg.n_layer):
        eng.k_cache[il][:S * ctx].copy_(torch.randn((S * ctx, eng.k_cache[il].shape[1]), device="cuda", generator=gen).half())
        eng.v_cache[il][:S * ctx].copy_(torch.randn((S * ctx, eng.v_cache[il].shape[1]), device="cuda", generator=gen).half())
    cells = torch.arange(S * ctx, device="cuda", dtype=torch.int32)
    eng.cell_seq[:S * ctx] = cells // ctx       # sequence s owns the contiguous run [s * ctx, (s + 1) * ctx)
    eng.cell_pos[:S * ctx] = cells % ctx
    seq = torch.arange(S, device="cuda", dtype=torch.int32)
    rng = np.random.default_rng(2)

    def step(i):
        eng.inp[0, :S] = torch.from_numpy(rng.integers(0, cfg.vocab, S).astype(np.int32)).cuda()
        eng.inp[1, :S] = ctx + i
        eng.inp[2, :S] = seq
        eng.inp[3, :S] = S * ctx + i * S + seq
        eng.run_device(S)

    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(3, 3 + a.reps):
        step(i)
    e1.record()
    e1.synchronize()
    ms = e0.elapsed_time(e1) / a.reps
    return {"kernel": "decode step", "layers": cfg.n_layer, "sequences": S, "context": ctx, "cells": n_cells, "ms_per_step": ms, "tok_s": S * 1e3 / ms,
            "launches_per_step": int(eng.launches_per_step[S]), "weight_GBps": cfg.weight_bytes_per_step() / ms / 1e6}


def run_umma_rate():
    """Builds csrc/probes/umma_rate.cu (a stand-alone program) next to the library and runs it; returns its report."""
    import os
    import subprocess

    from .build import CSRC, OUT, nvcc
    src, exe = os.path.join(CSRC, "probes", "umma_rate.cu"), os.path.join(OUT, "umma_rate")
    if not os.path.exists(exe) or os.path.getmtime(exe) < os.path.getmtime(src):
        os.makedirs(OUT, exist_ok=True)
        subprocess.check_call([nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-o", exe, src])
    return subprocess.run([exe], capture_output=True, text=True, timeout=120, check=True).stdout


def main():
    import sys
    if len(sys.argv) > 1 and sys.argv[1] == "umma-rate":
        print(run_umma_rate())
        return
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["mul_mat", "fattn", "quantize", "decode"])
    ap.add_argument("--ragged", action="store_true", help="fattn: the benchmark's ragged sequence lengths instead of --seqs x --ctx")
    ap.add_argument("--head-major", action="store_true", help="fattn: address the cache as [Hkv][cells][D] instead of the reference's [cells][Hkv][D]")
    ap.add_argument("--quant", action="store_true", help="fattn: b200_flash_attn_ext_quant (quantised output only)")
    ap.add_argument("--cfg2", choices=["a", "b"], default=None, help="fattn: the 16-sequence prefill ubatch (a: fits 8192 slots, b: cache enlarged)")
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--M", type=int, default=14336)
    ap.add_argument("--N", type=int, default=64)
    ap.add_argument("--wtype", type=int, default=2)
    ap.add_argument("--copies", type=int, default=8)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--seqs", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=900)
    ap.add_argument("--D", type=int, default=128)
    ap.add_argument("--H", type=int, default=32)
    ap.add_argument("--Hkv", type=int, default=8)
    ap.add_argument("--layers", type=int, default=32, help="decode: layers of the 8B architecture")
    ap.add_argument("--cells", type=int, default=8192, help="decode: cells of the unified cache (grown to what the sequences need)")
    a = ap.parse_args()
    fn = {"mul_mat": bench_mul_mat, "fattn": bench_fattn, "quantize": bench_quantize, "decode": bench_decode}[a.kernel]
    if a.kernel == "fattn" and a.cfg2:
        fn = bench_fattn_prefill
    r = fn(a)
    print(json.dumps(r))


if __name__ == "__main__":
    main()

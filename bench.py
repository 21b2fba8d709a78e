"""Benchmark: Q4_0 decode tok/s, Llama-3-8B architecture, 64 ragged sequences in a unified f16 KV cache of
65536 cells; mul_mat HBM GB/s against the measured peak.

    python bench.py --gpus 1 --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --steps K --warmup W    # the reference's ggml-cpu on the host cores

One "step" is one decode ubatch: every one of the 64 sequences advances by one token (32 layers of
quantised mul_mat + ragged flash attention + the small row ops, then the output head), i.e. 64 tokens.
With N > 1 (torchrun) every rank runs its own replica with its own 64 sequences (the 8B model fits one
GPU; there is no data-path collective), so the job is weak-scaled and `value` sums the ranks.  The same
line then carries a `rowsplit` record: ONE job of the 8B and of the 70B architecture whose mul_mat weights
are cut by rows over the N GPUs (strong scaling; at N = 1 the record holds the one-GPU time of the 70B
model the speed-ups refer to).

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from cactus_b200.workloads import N_CELLS, N_DECODE, N_SEQ, decode_attention_case, decode_step_inputs, prefilled_cells, prompt_lengths  # noqa: E402

METRIC = "Q4_0 decode tok/s (8B arch, 64 seqs)"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a timed region runs."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                for n, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# -------------------------------------------------------------------------------------------------
# CPU arm: the reference's own ggml-cpu (oracle/_ref) or, where that is absent, the plain-C port.
# -------------------------------------------------------------------------------------------------
def cpu_layer_sample(reps: int, warmup: int):
    """Times, on the host cores, the hot path of ONE layer of the 8B decode step at 64 columns (7 mul_mats
    + flash attention over the ragged cache) plus a 1/8 slice of the output head, and scales to the 32-layer step."""
    from cactus_b200.engine import LLAMA_3_8B as cfg
    from oracle.binding import Oracle, Q4_0, Reference
    ref = Reference.load(build=False)
    orc = Oracle()
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    rng = np.random.default_rng(0)
    lens, _ = prompt_lengths()
    t_layer = 0.0
    if ref is not None:
        kind, threads = "reference", cores
        for _, K, M in cfg.mul_mat_shapes():
            wq = rng.integers(0, 256, (M, K // 32 * 18), dtype=np.uint8)
            wq.reshape(M, K // 32, 18)[:, :, 1] = 0x1C   # fp16 scales ~ 2^-8
            x = rng.standard_normal((N_SEQ, K)).astype(np.float32)
            _, t = ref.mul_mat(Q4_0, wq, x, n_threads=threads, warmup=warmup, reps=reps)
            t_layer += t
        # attention: 64 decode tokens over a cache holding the 64 prompts
        c = decode_attention_case(lens, cfg)
        _, t = ref.flash_attn_ext(c["q"], c["kc"], c["vc"], c["mask"], c["scale"], n_kv=c["n_kv"], n_threads=threads, warmup=warmup, reps=reps)
        t_layer += t
        Mh = cfg.vocab // 8
        wq = rng.integers(0, 256, (Mh, cfg.d_model // 32 * 18), dtype=np.uint8)
        wq.reshape(Mh, cfg.d_model // 32, 18)[:, :, 1] = 0x1C
        _, t_head = ref.mul_mat(Q4_0, wq, rng.standard_normal((N_SEQ, cfg.d_model)).astype(np.float32), n_threads=threads, warmup=warmup, reps=reps)
        t_head *= 8
        sample = "1 of 32 layers (7 mul_mat at 64 columns + flash_attn over the 64-sequence cache) + 1/8 of the output head, scaled to the full step"
    else:
        kind, threads = "port", 1
        K, M = 4096, 4096
        wq = rng.integers(0, 256, (M // 8, K // 32 * 18), dtype=np.uint8)
        wq.reshape(M // 8, K // 32, 18)[:, :, 1] = 0x1C
        x = rng.standard_normal((N_SEQ, K)).astype(np.float32)
        t0 = time.perf_counter()
        orc.mul_mat(Q4_0, wq, x)
        t = (time.perf_counter() - t0) * 8
        macs_layer = sum(K * M for _, K, M in cfg.mul_mat_shapes())
        t_layer = t * macs_layer / (4096 * 4096)
        t_head = t * cfg.vocab * cfg.d_model / (4096 * 4096)
        sample = "1/8 of one 4096x4096 Q4_0 mul_mat at 64 columns with the scalar C port, scaled by MACs to the full step (attention not included)"
    step = cfg.n_layer * t_layer + t_head
    return {"value": N_SEQ / step, "unit": "tok/s", "cores": threads, "kind": kind, "sample": sample, "step_seconds": step}


# -------------------------------------------------------------------------------------------------
# GPU arm
# -------------------------------------------------------------------------------------------------
def ncu_dram_bytes_per_launch() -> dict:
    """DRAM bytes (read + write) per launch of the mul_mat at 64 columns, keyed by (K, M): ncu captures of
    `python -m cactus_b200.microbench mul_mat` on each of the step's shapes, kept with their commands in
    profiles/mul_mat_dram_bytes.json."""
    try:
        with open(os.path.join(ROOT, "profiles", "mul_mat_dram_bytes.json")) as f:
            return {(int(e["K"]), int(e["M"])): float(e["dram_bytes"]) for e in json.load(f)["launches"]}
    except (OSError, ValueError, KeyError):
        return {}


def mul_mat_roofline(eng, cfg, reps: int = 3):
    """Times the dominant kernel -- the Q4_0 mul_mat at 64 columns -- over all of the step's weights, launch
    by launch on the launching stream with CUDA events (weights of 32 distinct layers, 4.2 GB, so nothing is
    L2-resident), and relates the algorithmic bytes to the duration."""
    import torch
    from cactus_b200._lib import check, lib
    L = lib()
    names = {"wq": "attn_q", "wk": "attn_k", "wv": "attn_v", "wo": "attn_output", "gate": "ffn_gate", "up": "ffn_up", "down": "ffn_down"}
    T = N_SEQ
    per_shape, total_bytes, total_ms, launches = {}, 0.0, 0.0, 0
    per_layer = cfg.mul_mat_shapes()
    if eng.fused:   # the engine runs wq/wk/wv and gate/up as one stacked mul_mat each
        d, kvd, ff = cfg.d_model, cfg.n_kv_head * cfg.head_dim, cfg.d_ff
        names.update(qkv="attn_qkv", gate_up="ffn_gate_up")
        per_layer = [("qkv", d, d + 2 * kvd), ("wo", d, d), ("gate_up", d, 2 * ff), ("down", ff, d)]
    shapes = [(s, K, M, [f"blk.{il}.{names[s]}.weight" for il in range(cfg.n_layer)], cfg.layer_type) for s, K, M in per_layer]
    shapes.append(("output", cfg.d_model, cfg.vocab, ["output.weight"], cfg.head_type))
    for short, K, M, tensors, wtype in shapes:
        act = eng.act_ff if K == cfg.d_ff else eng.act_d
        out = {"qkv": getattr(eng, "qkv", None), "gate_up": getattr(eng, "gu", None), "output": eng.logits}.get(short)
        if out is None:
            out = {cfg.d_model: eng.tmp, cfg.d_ff: eng.gate, cfg.vocab: eng.logits}.get(M, eng.k)
        bb = 18 if wtype == 2 else 34
        n_products = {"qkv": 3, "gate_up": 2}.get(short, 1)       # the reference's mul_mats behind this launch: each reads the activations
        alg = M * (K // 32) * bb + n_products * T * K * 4 + T * M * 4      # weights + f32 activations in + f32 out
        def launch_all():
            stq = torch.cuda.current_stream().cuda_stream
            for name in tensors:
                w = eng.w.tensors[name]
                check(L.b200_mul_mat_q_prequant(w.wtype, w.data.data_ptr(), w.K, w.M, act.data_ptr(), T, out.data_ptr(), out.stride(0) * 4,
                                                eng.ws.data_ptr(), eng.ws.numel(), stq))

        launch_all()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            launch_all()
        best = None
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            e1.synchronize()
            ms = e0.elapsed_time(e1) / len(tensors)
            best = ms if best is None else min(best, ms)
        per_shape[short] = {"K": K, "M": M, "ms": round(best, 5), "GBps": round(alg / best / 1e6, 1)}
        total_bytes += alg * len(tensors)
        total_ms += best * len(tensors)
        launches += len(tensors)
    peak, which = peaks()
    achieved = total_bytes / total_ms / 1e6
    traffic = None
    table = ncu_dram_bytes_per_launch()
    if all((K, M) in table for _, K, M, _, _ in shapes):
        traffic = int(sum(table[(K, M)] * len(t) for _, K, M, t, _ in shapes))
    return {"bound": "hbm", "kernel": "mmq_kernel<Q4_0,64> (all mul_mat launches of one decode step)", "achieved": round(achieved, 1),
            "peak": peak, "peak_source": which, "unit": "GB/s", "frac": round(achieved / peak, 4), "traffic": traffic,
            "algorithmic_bytes_per_step": int(total_bytes), "ms_per_step_in_mul_mat": round(total_ms, 4), "per_shape": per_shape}


def fill_prompt_cells(eng, head: int, seed: int):
    """The prefilled prompts: synthetic K/V ~ N(0, 1) in the cells the prompts own."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(seed)
    for il in range(eng.cfg.n_layer):
        eng.k_cache[il][:head].copy_(torch.randn((head, eng.k_cache[il].shape[1]), device="cuda", generator=gen).half())
        eng.v_cache[il][:head].copy_(torch.randn((head, eng.v_cache[il].shape[1]), device="cuda", generator=gen).half())


def time_decode_steps(eng, steps_dev, cp0, cs0, K: int, W: int, local: int):
    """Device time (ms, maximum over the ranks) of K decode ubatches after W untimed ones, inputs resident in HBM;
    clocks sampled during the timed region."""
    import torch
    from cactus_b200 import dist as bdist

    def barrier():
        torch.cuda.synchronize()
        bdist.barrier()
        torch.cuda.synchronize()

    eng.cell_pos.copy_(cp0)
    eng.cell_seq.copy_(cs0)
    for s in range(W):
        eng.inp.copy_(steps_dev[s])
        eng.run_device(N_SEQ)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(W, W + K):
        if s % N_DECODE == 0:
            eng.cell_pos.copy_(cp0)
            eng.cell_seq.copy_(cs0)
        eng.inp.copy_(steps_dev[s])
        eng.run_device(N_SEQ)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    return bdist.max_over_ranks(ms, "cuda"), clocks


def rowsplit_record(model: str, rank: int, world: int, local: int, lens, head, cp0, cs0, steps_dev, K: int, W: int):
    """ONE job of `model` on `world` GPUs: every mul_mat weight cut by rows, joined after every product (with one GPU:
    the plain engine -- the time the speed-ups of the sharded runs refer to)."""
    import gc

    import torch
    from cactus_b200.engine import LLAMA_3_8B, LLAMA_3_70B, LlamaEngine, LlamaWeights
    from cactus_b200.rowsplit import RowSplit
    cfg = LLAMA_3_70B if model == "70b" else LLAMA_3_8B
    split = RowSplit(rank, world, 128 << 20) if world > 1 else None
    weights = LlamaWeights.random(cfg, seed=0, rank=rank, world=world)
    eng = LlamaEngine(weights, N_CELLS, max_tokens=N_SEQ, split=split)
    fill_prompt_cells(eng, head, 100)
    ms, clocks = time_decode_steps(eng, steps_dev, cp0, cs0, K, W, local)
    status = split.status() if split is not None else 0
    per_gpu_weight_bytes = cfg.weight_bytes_per_step() / world
    peak, _ = peaks()
    rec = {"n_gpus": world, "ms_per_step": round(ms / K, 4), "tok_s": round(N_SEQ * K / (ms / 1e3), 1), "peer_status": status, "steps": K,
           "launches_per_step": int(eng.launches_per_step[N_SEQ]), "head_parallel_attention": bool(eng.hp),
           "weight_stream_frac_of_hbm_peak": round(per_gpu_weight_bytes / (ms / K / 1e3) / 1e9 / peak, 4), "sm_mhz": clocks.get("sm_mhz")}
    del eng, weights
    if split is not None:
        split.close()
    gc.collect()
    torch.cuda.empty_cache()
    return rec


def other_configs(L, local: int):
    """The smaller workloads of the hot path, each timed on the device: the single 4096 x 4096 Q4_0 mul_mat at 1, 8 and
    512 columns (distinct weight copies larger than L2 in turn), the single FLASH_ATTN_EXT op on a ragged 16-sequence
    ubatch over an 8192-slot cache, and the 1B architecture with one sequence: a 512-token prompt ubatch, then decode."""
    from types import SimpleNamespace

    import torch
    from cactus_b200 import microbench
    from cactus_b200.engine import LLAMA_32_1B, LlamaEngine, LlamaWeights
    peak, _ = peaks()
    out = {"mul_mat_4096x4096_q4_0": {}}
    for N in (1, 8, 512):
        r = microbench.bench_mul_mat(SimpleNamespace(K=4096, M=4096, N=N, wtype=2, copies=24, reps=5))
        out["mul_mat_4096x4096_q4_0"][f"N={N}"] = {"us": round(r["ms_per_launch"] * 1e3, 2), "GBps": round(r["GBps"], 1), "frac_of_hbm_peak": round(r["GBps"] / peak, 3),
                                                    "TOPS": round(r["TOPS"], 1)}
    r = microbench.bench_fattn_prefill(SimpleNamespace(D=128, H=32, Hkv=8, cfg2="a", copies=8, reps=5))
    out["flash_attn_16seq_ubatch_8192_slots"] = {"us": round(r["ms_per_launch"] * 1e3, 1), "query_tokens": r["tokens"], "attended_pairs": r["attended_pairs"],
                                                  "TFLOPs": round(r["TFLOPs"], 1), "GBps": round(r["GBps"], 1), "frac_of_hbm_peak": round(r["GBps"] / peak, 3)}
    cfg = LLAMA_32_1B
    # the prompt as one 512-token ubatch through the public call (host inputs, the step, greedy ids back)
    import numpy as np
    eng = LlamaEngine(LlamaWeights.random(cfg, seed=3), 1024, max_tokens=512, use_graphs=False)
    rng = np.random.default_rng(0)
    toks, pos, seq, slots = rng.integers(0, cfg.vocab, 512), np.arange(512), np.zeros(512, np.int64), np.arange(512)
    eng.decode(toks, pos, seq, slots, want_logits=False)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        eng.decode(toks, pos, seq, slots, want_logits=False)
    e1.record()
    e1.synchronize()
    ms_prompt = e0.elapsed_time(e1) / 3
    out["llama_1b_prompt_512_tokens"] = {"ms": round(ms_prompt, 3), "tok_s": round(512 / (ms_prompt / 1e3), 1), "includes": "H2D of the inputs, all 512 rows of the output head, greedy ids D2H (no logits read-back)"}
    del eng
    torch.cuda.empty_cache()
    eng = LlamaEngine(LlamaWeights.random(cfg, seed=3), 1024, max_tokens=8)
    n_prompt = 512
    eng.cell_pos[:n_prompt] = torch.arange(n_prompt, dtype=torch.int32, device="cuda")
    eng.cell_seq[:n_prompt] = 0
    fill_prompt_cells(eng, n_prompt, 5)
    steps = 64
    for s in range(steps + 5):
        if s == 5:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        eng.inp[:, 0] = torch.tensor([s % cfg.vocab, n_prompt + s, 0, n_prompt + s], dtype=torch.int32, device="cuda")
        eng.run_device(1)
    e1.record()
    e1.synchronize()
    ms = e0.elapsed_time(e1) / steps
    out["llama_1b_one_sequence_decode"] = {"ms_per_token": round(ms, 4), "tok_s": round(1e3 / ms, 1), "context": n_prompt,
                                           "weight_stream_frac_of_hbm_peak": round(cfg.weight_bytes_per_step() / (ms / 1e3) / 1e9 / peak, 3),
                                           "launches_per_token": int(eng.launches_per_step[1])}
    del eng
    torch.cuda.empty_cache()
    return out


def plugin_record():
    """The same decode step through the drop-in itself: the ggml backend plug-in driven by the reference's unchanged
    llama_decode (tests/_bin/harness, built where a checkout of the reference is present; it travels as a binary with the
    reference's runtime compiled into oracle/_ref).  Synthetic 8B GGUF written to /tmp, 64 sequences with random prompts
    in a 65536-cell cache, then timed 64-token decode batches; the KQ mask is synthesised on the device (the driver's
    replacement of set_input_kq_mask hands the cell metadata to the backend's extension proc)."""
    harness = os.path.join(ROOT, "tests", "_bin", "harness")
    if not os.path.exists(harness):
        return {"unavailable": "tests/_bin/harness was not built (needs a checkout of the reference at build time)"}
    cmd = [harness, "model", "--layers", "32", "--d", "4096", "--heads", "32", "--kv", "8", "--ff", "14336", "--vocab", "128256", "--ctx", "65536",
           "--seqs", "64", "--max-prompt", "1790", "--skip-cpu", "--head-q4", "--bench-steps", "10", "--decode", "2", "--device-mask", "--path", "/tmp/b200_bench_8b.gguf"]
    try:
        p = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=dict(os.environ, B200_TIMING="1"))
        r = [json.loads(line) for line in p.stdout.splitlines() if line.startswith("{")][-1]
    except (subprocess.SubprocessError, IndexError, ValueError, OSError) as e:
        return {"unavailable": f"harness run failed: {e!r}"[:200]}
    if "error" in r:
        return {"unavailable": str(r)[:200]}
    return {"path": "llama_decode (reference runtime, unchanged) -> scheduler -> libggml-b200.so graph_compute -> C ABI", "ms_per_step_wall": r["b200_step_ms"],
            "tok_s": round(N_SEQ / (r["b200_step_ms"] / 1e3), 1), "device_ms_per_step": r["device_ms_per_graph"], "device_side_masks": r["device_masks"],
            "logits": "full 64 x 128256 f32 read back into the context's pinned buffer every step (32.8 MB: most of wall minus device time)",
            "graphs_recorded": r.get("graphs_recorded"), "graphs_replayed": r.get("graphs_replayed"), "steps": 10}


def gpu_arm(args):
    import gc

    import torch

    from cactus_b200 import dist as bdist
    from cactus_b200 import lib
    from cactus_b200.engine import LLAMA_3_8B, LLAMA_3_70B, LlamaConfig, LlamaEngine, LlamaWeights
    from cactus_b200.rowsplit import RowSplit

    rank, world, local = bdist.env_rank()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    bdist.init("nccl", torch.device("cuda", local))
    L = lib()

    cfg = LlamaConfig(4, 1024, 8, 2, 4096, 32000) if args.small else (LLAMA_3_70B if args.model == "70b" else LLAMA_3_8B)
    lens, scale = prompt_lengths()
    cell_pos, cell_seq, head = prefilled_cells(lens)
    rows = args.split == "rows" and world > 1
    if rows:   # one job: every rank holds its rows of the weights and the whole (replicated) KV cache and activations
        split = RowSplit(rank, world, 128 << 20)
        weights = LlamaWeights.random(cfg, seed=0, rank=rank, world=world)
        eng = LlamaEngine(weights, N_CELLS, max_tokens=N_SEQ, split=split)
    else:
        split = None
        weights = LlamaWeights.random(cfg, seed=rank)
        eng = LlamaEngine(weights, N_CELLS, max_tokens=N_SEQ)
    jobs = 1 if rows else world
    fill_prompt_cells(eng, head, 100 + (0 if rows else rank))
    cp0, cs0 = torch.from_numpy(cell_pos).cuda(), torch.from_numpy(cell_seq).cuda()

    def reset_state():
        eng.cell_pos.copy_(cp0)
        eng.cell_seq.copy_(cs0)

    def barrier():
        torch.cuda.synchronize()
        bdist.barrier()
        torch.cuda.synchronize()

    K, W = args.steps, max(args.warmup, 3)
    assert K >= 1
    total = W + K
    steps_dev = torch.from_numpy(np.stack([np.stack(decode_step_inputs(lens, head, s % N_DECODE)) for s in range(total)])).cuda()  # [total,4,64]

    # ---- value: inputs resident in HBM, device-timed ---------------------------------------------
    ms_max, clocks = time_decode_steps(eng, steps_dev, cp0, cs0, K, W, local)
    launches0 = eng.launches_per_step[N_SEQ]
    value = jobs * N_SEQ * K / (ms_max / 1e3)

    # ---- e2e: the public call with host buffers, H2D of the inputs and D2H of the logits inside ---
    def e2e_leg(want_logits: bool):
        reset_state()
        tok = None
        n = min(K, N_DECODE - W)
        for s in range(W):
            _, tok = eng.decode(*decode_step_inputs(lens, head, s, tokens=tok), want_logits=want_logits)
        barrier()
        t0 = time.perf_counter()
        for s in range(W, W + n):
            _, tok = eng.decode(*decode_step_inputs(lens, head, s, tokens=tok), want_logits=want_logits)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        return bdist.job_throughput(N_SEQ * n, dt, "cuda") * jobs / world, n

    e2e, e2e_steps = e2e_leg(True)
    e2e_ids, _ = e2e_leg(False)     # the greedy ids only (b200_argmax_rows on the device): what the 32.8 MB logits read-back costs
    h2d = 4 * N_SEQ * 4
    d2h = N_SEQ * cfg.vocab * 4 + N_SEQ * 4

    # ---- one sequence decoding alone on the same engine (the GEMV path): device-timed, inputs resident ----
    one_seq = None
    if rank == 0 and world == 1 and not rows and not args.small and not args.no_extras:
        reset_state()
        longest = int(np.argmax(lens))
        n1 = 32
        for s in range(n1 + 3):
            if s == 3:
                torch.cuda.synchronize()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
            tok, pos, seq, slots = decode_step_inputs(lens, head, s)
            eng.inp[:, 0] = torch.tensor([int(tok[longest]), int(pos[longest]), int(seq[longest]), int(slots[longest])], dtype=torch.int32, device="cuda")
            eng.run_device(1)
        t1.record()
        t1.synchronize()
        ms1 = t0.elapsed_time(t1) / n1
        one_seq = {"ms_per_token": round(ms1, 4), "tok_s": round(1e3 / ms1, 1), "context": int(lens[longest]),
                   "weight_stream_frac_of_hbm_peak": round(cfg.weight_bytes_per_step() / (ms1 / 1e3) / 1e9 / peaks()[0], 3),
                   "launches_per_token": int(eng.launches_per_step[1])}

    roof = mul_mat_roofline(eng, cfg) if (rank == 0 and not rows) else None
    peer_status = split.status() if rows else 0
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_layer_sample(reps=2, warmup=1)

    # ---- the sharded job (row split) on the same GPUs, and the smaller workloads --------------------------------
    del eng, weights
    if rows:
        split.close()
    gc.collect()
    torch.cuda.empty_cache()
    rowsplit = None
    if not args.small and not args.no_extras:
        Kr = min(K, 10)
        rowsplit = {"what": "ONE job per model on all GPUs of the run: mul_mat weights cut by rows, every product joined over NVLink "
                            "(strong scaling); n_gpus 1 = the plain engine"}
        for model in (("8b", "70b") if world > 1 else ("70b",)):
            rowsplit[model] = rowsplit_record(model, rank, world, local, lens, head, cp0, cs0, steps_dev, Kr, W)
        if world == 1:
            rowsplit["8b"] = {"n_gpus": 1, "ms_per_step": round(ms_max / K, 4), "tok_s": round(value, 1), "peer_status": 0, "steps": K}
    extras = other_configs(L, local) if (rank == 0 and world == 1 and not args.small and not args.no_extras) else None
    if extras is not None and one_seq is not None:
        extras["llama_8b_one_sequence_decode"] = one_seq
    plugin = plugin_record() if (rank == 0 and world == 1 and not args.small and not args.no_extras) else None

    if rank == 0:
        kv_bytes = int(lens.sum() + N_SEQ * (W + K / 2)) * cfg.n_layer * 2 * cfg.n_kv_head * cfg.head_dim * 2
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": round(ms_max / K, 4), "higher_is_better": True, "scaling": "strong" if rows else "weak", "vs_baseline": None,
            "dtype": "int8 x int4/int8 block dots, f32 accumulate; f16 KV", "data": "synthetic",
            "config": {"workload": ("Llama-3-70B architecture" if args.model == "70b" and not args.small else "Llama-3-8B architecture") +
                                   ", random N(0,0.02) weights in Q4_0, continuous batching of 64 sequences in a unified f16 KV cache of 65536 cells, "
                                   "one decode ubatch of 64 tokens per step",
                       "prompt_lengths": f"U[16,2048] seed 0 scaled by {scale:.3f} to leave 128 decode cells per sequence; "
                                         f"{int(lens.sum())} prompt cells hold synthetic N(0,1) K/V",
                       "parallelism": (f"row split over {world} GPUs: every mul_mat weight cut by rows, the products' own write-back stores into every GPU's "
                                       f"buffers over NVLink (b200_mul_mat_q_rowsplit / _stacked); attention, rope and the KV cache follow the heads of a rank "
                                       f"(attention output joined with b200_allgather_rows), norms replicated; peer_status {peer_status}") if rows
                                      else ("one replica per GPU, no collective (the row split of the same GPUs is in `rowsplit`)" if world > 1 else "single GPU"),
                       "model": args.model if not args.small else "small",
                       "l2": "inputs larger than L2: 4.2 GB of weights and ~7 GB of KV are streamed every step"},
            "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "ids_only": {"value": round(e2e_ids, 1), "unit": "tok/s", "d2h_bytes_per_step": N_SEQ * 4}},
            "gpu_launches": int(launches0 * K), "launches_per_step": int(launches0),
            "clocks": clocks, "roofline": roof, "cpu_baseline": cpu,
            "step_bytes": {"weights": cfg.weight_bytes_per_step(), "kv_read_about": kv_bytes},
            "rowsplit": rowsplit, "other_configs": extras, "plugin": plugin,
        }
        print(json.dumps(line))
    bdist.shutdown()


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    K, W = args.steps, args.warmup
    reps = max(1, min(K, 5))
    t0 = time.perf_counter()
    r = cpu_layer_sample(reps=reps, warmup=min(W, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": round(r["value"], 3), "unit": "tok/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": K, "warmup": W, "ms_per_step": round(r["step_seconds"] * 1e3, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int4 block dots (AVX2), f32 accumulate", "data": "synthetic",
        "config": {"workload": "Llama-3-8B architecture, Q4_0, decode ubatch of 64 tokens over the 64-sequence cache: reference ggml-cpu on the host cores, timed on a bounded sample",
                   "sample": r["sample"], "timed_reps_per_op": reps, "wall_seconds": None},
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": round(r["value"], 3), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    line["config"]["wall_seconds"] = round(time.perf_counter() - t0, 1)
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--small", action="store_true", help="a small model for debugging the harness (not a bench number)")
    ap.add_argument("--split", default="none", choices=["none", "rows"],
                    help="rows: ONE job whose mul_mat weights are row-split over the GPUs and joined after every product (strong scaling); "
                         "none: one replica per GPU (weak scaling, the default)")
    ap.add_argument("--model", default="8b", choices=["8b", "70b"], help="70b: the Llama-3-70B architecture on the same 64-sequence workload")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the row-split record and the smaller workloads")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()

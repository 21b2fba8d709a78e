"""Synthetic workloads of the benchmark (numpy only): the continuous-batching serving state -- 64 sequences with ragged
prompts of up to 1024 tokens in a unified KV cache of 65536 cells -- after the prompts have been prefilled."""
from __future__ import annotations

import numpy as np

N_SEQ = 64
N_CELLS = 65536
N_DECODE = 128


def prompt_lengths(seed: int = 0):
    """Prompt lengths ~ U[16, 2048] for 64 sequences.  As drawn they need more cells than the 65536-cell
    cache has once 128 decode tokens per sequence are added, so they are scaled down proportionally."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(16, 2049, N_SEQ)
    budget = N_CELLS - N_SEQ * N_DECODE
    scale = min(1.0, budget / lens.sum())
    lens = np.maximum(16, np.floor(lens * scale).astype(np.int64))
    while lens.sum() > budget:
        lens[np.argmax(lens)] -= 1
    return lens, float(scale)


def prefilled_cells(lens):
    """Cell metadata after the prompts were prefilled in order: sequence s owns a contiguous run (the
    reference's find_slot hands out contiguous runs per ubatch, cactus/llama-kv-cache.cpp:476-569)."""
    cell_pos = np.full(N_CELLS, -1, np.int32)
    cell_seq = np.full(N_CELLS, -1, np.int32)
    head = 0
    for s, n in enumerate(lens):
        cell_pos[head:head + n] = np.arange(n)
        cell_seq[head:head + n] = s
        head += n
    return cell_pos, cell_seq, head


def decode_step_inputs(lens, head, step, tokens=None, seed=1):
    """(tokens, pos, seq, slots) of decode step `step`: one token per sequence, 64 fresh contiguous cells."""
    rng = np.random.default_rng([seed, step])
    tok = rng.integers(0, 128256, N_SEQ).astype(np.int32) if tokens is None else np.asarray(tokens, np.int32)
    pos = (np.asarray(lens) + step).astype(np.int32)
    seq = np.arange(N_SEQ, dtype=np.int32)
    slots = (head + step * N_SEQ + np.arange(N_SEQ)).astype(np.int32)
    return tok, pos, seq, slots


def decode_attention_case(lens, cfg, seed=2):
    """Host-side FLASH_ATTN_EXT inputs of the first decode step over the prefilled cache (for the CPU arm)."""
    rng = np.random.default_rng(seed)
    cell_pos, cell_seq, head = prefilled_cells(lens)
    tok, pos, seq, slots = decode_step_inputs(lens, head, 0)
    cell_pos[slots] = pos
    cell_seq[slots] = seq
    n_kv = (head + N_SEQ + 255) // 256 * 256
    D, H, Hkv = cfg.head_dim, cfg.n_head, cfg.n_kv_head
    kc = rng.integers(0x3000, 0x3C00, (n_kv, Hkv, D), dtype=np.uint16)   # positive f16 values in [0.125, 1)
    vc = rng.integers(0x3000, 0x3C00, (n_kv, Hkv, D), dtype=np.uint16)
    q = rng.standard_normal((N_SEQ, H, D)).astype(np.float32)
    ok = (cell_seq[None, :n_kv] == seq[:, None]) & (cell_pos[None, :n_kv] <= pos[:, None])
    mask = np.full((64, n_kv), 0xFC00, np.uint16)
    mask[ok] = 0
    return dict(q=q, kc=kc, vc=vc, mask=mask, n_kv=int(n_kv), scale=float(D) ** -0.5)

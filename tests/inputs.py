"""Seeded synthetic inputs shared by the golden-vector generator and the tests.

Everything is derived from numpy's PCG64 ``default_rng`` streams, which are stable across numpy
versions, so the golden file stores outputs only.
"""
from __future__ import annotations

import zlib

import numpy as np

CFG1_SAMPLE_STRIDE = 61  # column sample of the 512-column config-1 output kept in the golden file


def checksum(a: np.ndarray) -> int:
    return zlib.crc32(np.ascontiguousarray(a).view(np.uint8).tobytes())


# ---- quantiser ------------------------------------------------------------------------------------
def quantizer_rows() -> np.ndarray:
    """[56, 512] f32: gaussian rows plus the edge cases of quantize_row_q8_0 (zeros, ties, tiny, huge)."""
    rng = np.random.default_rng(100)
    K = 512
    rows = [rng.standard_normal((40, K)).astype(np.float32)]
    rows.append(np.zeros((1, K), np.float32))
    tie = np.tile(np.arange(-16, 16, dtype=np.float32) + 0.5, K // 32)  # k+0.5 with amax forced to 127 -> id = 1
    tie = tie.reshape(K // 32, 32)
    tie[:, 0] = 127.0
    rows.append(tie.reshape(1, K))
    tie2 = -tie.copy()
    rows.append(tie2.reshape(1, K))
    rows.append((rng.standard_normal((2, K)) * 1e-30).astype(np.float32))  # fp16 scale underflows to subnormal / zero
    rows.append((rng.standard_normal((2, K)) * 3e4).astype(np.float32))
    rows.append((rng.standard_normal((2, K)) * 1e-3).astype(np.float32))
    spike = np.zeros((1, K), np.float32)
    spike[0, ::37] = -5.0
    rows.append(spike)
    rows.append(rng.uniform(-1, 1, (6, K)).astype(np.float32))
    return np.concatenate(rows, 0)


def small_weights() -> np.ndarray:
    rng = np.random.default_rng(101)
    w = (rng.standard_normal((24, 256)) * 0.02).astype(np.float32)
    w[5] = 0.0
    w[6, :32] = 0.0
    return w


def small_activations() -> np.ndarray:
    rng = np.random.default_rng(102)
    x = rng.standard_normal((5, 256)).astype(np.float32)
    x[3, 32:64] = 0.0
    return x


# ---- config 1: Q4_0 [4096 out x 4096 in], activations N(0,1) [N x 4096], seed 0 ---------------------
def cfg1_weights() -> np.ndarray:
    return (np.random.default_rng(0).standard_normal((4096, 4096)) * 0.02).astype(np.float32)


def cfg1_activations(N: int) -> np.ndarray:
    return np.random.default_rng([0, N]).standard_normal((N, 4096)).astype(np.float32)


def head_weights() -> np.ndarray:
    return (np.random.default_rng(103).standard_normal((512, 2048)) * 0.02).astype(np.float32)


def head_activations() -> np.ndarray:
    return np.random.default_rng(104).standard_normal((3, 2048)).astype(np.float32)


# ---- ragged multi-sequence attention -----------------------------------------------------------------
def ragged_case(seed: int, D: int, H: int, Hkv: int, n_cells: int, seqs, shuffle=True, pad=256):
    """Unified-cache attention inputs.

    ``seqs`` is a list of (context_length, n_query_tokens): each sequence owns a contiguous run of
    ``context_length`` cells (runs placed in random sequence order) holding positions 0..ctx-1; its query
    tokens are the last ``n_query_tokens`` positions (their K/V are already in the cache, as in the
    reference where find_slot runs before the mask is built).  Tokens of different sequences are
    interleaved in the ubatch in sequence order.  Returns a dict with q [Nq,H,D] f32, kc/vc uint16 (f16
    bits) [n_cells,Hkv,D], mask uint16 [pad64(Nq), n_kv], n_kv (padded to ``pad``), scale, and the
    metadata (cell_pos, cell_seq, tok_pos, tok_seq).
    """
    rng = np.random.default_rng(seed)
    order = rng.permutation(len(seqs)) if shuffle else np.arange(len(seqs))
    cell_pos = np.full(n_cells, -1, np.int32)
    cell_seq = np.full(n_cells, -1, np.int32)
    head = 0
    for s in order:
        ctx, _ = seqs[s]
        assert head + ctx <= n_cells, "sequences do not fit the cache"
        cell_pos[head:head + ctx] = np.arange(ctx)
        cell_seq[head:head + ctx] = s
        head += ctx
    n_kv = min(n_cells, max(pad, (head + pad - 1) // pad * pad))
    tok_pos, tok_seq = [], []
    for s, (ctx, nq) in enumerate(seqs):
        tok_pos += list(range(ctx - nq, ctx))
        tok_seq += [s] * nq
    tok_pos = np.array(tok_pos, np.int32)
    tok_seq = np.array(tok_seq, np.int32)
    Nq = len(tok_pos)
    q = rng.standard_normal((Nq, H, D)).astype(np.float32)
    kc = rng.standard_normal((n_cells, Hkv, D)).astype(np.float16).view(np.uint16)
    vc = rng.standard_normal((n_cells, Hkv, D)).astype(np.float16).view(np.uint16)
    Np = (Nq + 63) // 64 * 64
    ok = (cell_seq[None, :n_kv] == tok_seq[:, None]) & (cell_pos[None, :n_kv] <= tok_pos[:, None]) & (cell_seq[None, :n_kv] >= 0)
    mask = np.full((Np, n_kv), 0xFC00, np.uint16)
    mask[:Nq][ok] = 0
    return dict(q=q, kc=kc, vc=vc, mask=mask, n_kv=int(n_kv), scale=float(1.0 / np.sqrt(D)), cell_pos=cell_pos,
                cell_seq=cell_seq, tok_pos=tok_pos, tok_seq=tok_seq, valid_rows=np.arange(Nq), D=D, H=H, Hkv=Hkv)


def fattn_cases():
    cases = {
        "d128_gqa4": ragged_case(200, 128, 32, 8, 768, [(300, 3), (17, 1), (200, 5)]),
        "d64_gqa4": ragged_case(201, 64, 8, 2, 256, [(100, 4), (60, 1), (1, 1)]),
        "d128_gqa8_decode": ragged_case(202, 128, 16, 2, 1024, [(257, 1), (500, 1), (31, 1), (64, 1)]),
        "d128_prefill": ragged_case(203, 128, 8, 2, 512, [(130, 130)]),
    }
    c = ragged_case(204, 128, 8, 8, 256, [(90, 2), (40, 3)])
    c["softcap"] = 30.0
    cases["softcap"] = c
    c = ragged_case(205, 64, 12, 4, 256, [(77, 2), (128, 1)])
    c["max_bias"] = 8.0
    cases["alibi"] = c
    return cases


def row_op_inputs():
    rng = np.random.default_rng(300)
    return dict(
        x=rng.standard_normal((7, 2048)).astype(np.float32),
        y=rng.standard_normal((7, 2048)).astype(np.float32),
        w=(1.0 + 0.1 * rng.standard_normal(2048)).astype(np.float32),
        xr=rng.standard_normal((7, 4, 128)).astype(np.float32),
        pos=np.array([0, 1, 5, 100, 4095, 70000, 3], np.int32),
        # K-shift of cached keys: f16 rows [cells, kv heads, D] and a per-cell position shift (zero, negative, large)
        kf16=rng.standard_normal((9, 2, 128)).astype(np.float16).view(np.uint16),
        shift=np.array([0, -1, 7, -512, 0, 2048, -33000, 1, 0], np.int32),
    )

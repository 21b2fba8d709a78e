"""FLASH_ATTN_EXT for ubatches with many query tokens: the query-tiled kernel (a CTA per tile of consecutive tokens and
kv-head, K/V chunks staged once per tile) against the oracle, on every token.

Same tolerances as test_gpu_fattn.py: <= 1e-5 of the double-accumulated result, and no further from the reference than
2e-3 plus the reference's own distance from that result."""
import numpy as np
import pytest

import inputs
from gpu_util import dev, f16, host, rel_max_err

pytestmark = pytest.mark.gpu
TOL = 2e-3


def run_case(c):
    from cactus_b200 import ops
    return host(ops.flash_attn_ext(dev(c["q"]), f16(c["kc"]), f16(c["vc"]), f16(c["mask"]), c["scale"], n_kv=c["n_kv"]))


def check(oracle, c, every=1):
    got = run_case(c)
    rows = np.arange(0, len(c["tok_pos"]), every)
    Np = (len(rows) + 63) // 64 * 64
    maskp = np.full((Np, c["n_kv"]), 0xFC00, np.uint16)
    maskp[:len(rows)] = c["mask"][rows]
    ref = oracle.flash_attn_ext(c["q"][rows], c["kc"], c["vc"], maskp, c["scale"], n_kv=c["n_kv"])[:len(rows)]
    truth = oracle.flash_attn_ext(c["q"][rows], c["kc"], c["vc"], maskp, c["scale"], n_kv=c["n_kv"], acc_mode=1)[:len(rows)]
    assert np.isfinite(got).all()
    assert rel_max_err(got[rows], truth) < 1e-5
    assert rel_max_err(got[rows], ref) < TOL + rel_max_err(ref, truth)


@pytest.mark.parametrize("spec", [
    (128, 32, 8, 2048, [(900, 200), (300, 56)]),          # two prompts, GQA 4: 16-token tiles, one tile straddles the sequences
    (128, 64, 8, 1024, [(600, 130)]),                     # GQA 8 (70B architecture): 8-token tiles, ragged last tile
    (64, 32, 8, 1024, [(512, 128), (200, 40)]),           # head size 64 (1B architecture)
    (128, 4, 4, 512, [(300, 150)]),                       # no GQA: 64-token tiles
    (128, 8, 2, 1024, [(400, 129), (50, 1), (120, 7)]),   # a prompt, a decode token and a short chunk in one ubatch
])
def test_prefill_ubatches_vs_oracle_every_token(oracle, spec):
    D, H, Hkv, cells, seqs = spec
    c = inputs.ragged_case(sum(n for _, n in seqs), D, H, Hkv, cells, seqs)
    assert len(c["tok_pos"]) >= 128
    check(oracle, c)


def test_512_token_ubatch_of_16_ragged_sequences_every_token(oracle):
    """16 sequences with contexts from U[64, 4096] (rescaled to 8192 slots) and 1-256 query tokens each, clipped to a
    512-token ubatch: every token against the oracle."""
    rng = np.random.default_rng(0)
    ctx = rng.integers(64, 4097, 16)
    nq = rng.integers(1, 257, 16)
    ctx = np.maximum(64, (ctx * min(1.0, 8192 / ctx.sum() * 0.999)).astype(int))
    while ctx.sum() > 8192:
        ctx[np.argmax(ctx)] -= ctx.sum() - 8192
    nq = np.minimum(nq, ctx)
    nq = np.maximum(1, (nq * min(1.0, 512 / nq.sum())).astype(int))
    c = inputs.ragged_case(0, 128, 32, 8, 8192, list(zip(ctx.tolist(), nq.tolist())))
    check(oracle, c)


def test_decode_batch_of_many_sequences_keeps_the_per_token_kernel(oracle):
    """160 tokens of 160 different sequences share no cells: the plan built with the mask index sends the ubatch to the
    per-token kernel (both are launched, one returns at once); results as ever."""
    seqs = [(20 + (7 * i) % 40, 1) for i in range(160)]
    c = inputs.ragged_case(3, 128, 8, 2, 8192, seqs)
    check(oracle, c)


def test_tiled_and_per_token_kernels_agree():
    """The same prefill ubatch through both kernels (B200_FA_TILE_MIN_NQ=0 in a child process turns the tiled one off)."""
    import json
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    code = f"""
import sys, json
sys.path.insert(0, {here!r}); sys.path.insert(0, {os.path.dirname(here)!r})
import numpy as np, inputs
from gpu_util import dev, f16, host
from cactus_b200 import ops
c = inputs.ragged_case(11, 128, 32, 8, 4096, [(1500, 300), (700, 90)])
out = host(ops.flash_attn_ext(dev(c["q"]), f16(c["kc"]), f16(c["vc"]), f16(c["mask"]), c["scale"], n_kv=c["n_kv"]))
np.save(sys.argv[1], out)
"""
    outs = []
    for i, env in enumerate(({}, {"B200_FA_TILE_MIN_NQ": "0"})):
        path = f"/tmp/b200_fa_tile_{os.getpid()}_{i}.npy"
        r = subprocess.run([sys.executable, "-c", code, path], env=dict(os.environ, **env), capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        outs.append(np.load(path))
        os.remove(path)
    assert rel_max_err(outs[0], outs[1]) < 1e-5

"""The tcgen05 (TMEM accumulator) mul_mat kernels against the oracle.

A kernel is selected per process (B200_MMQ_TC=1: block dots on the tensor core, scales in the epilogue; 2: scales folded
into fp16 operands, three product terms; 3: the same with two terms), so each case runs in a child interpreter; the
child prints the relative error and the library's kernel status (non-zero after a bounded barrier wait gave up).
"""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

CHILD = r"""
import json, sys
sys.path.insert(0, {here!r}); sys.path.insert(0, {root!r})
import numpy as np, torch
from oracle.binding import Oracle, Q4_0, Q8_0
from cactus_b200 import ops, _lib
o = Oracle()
out = []
for (wtype, M, K, N) in {cases!r}:
    rng = np.random.default_rng(M + K + N)
    wq = o.quantize_weights(wtype, (rng.standard_normal((M, K)) * 0.02).astype(np.float32))
    x = rng.standard_normal((N, K)).astype(np.float32)
    ref, _ = o.mul_mat(wtype, wq, x)
    got = ops.mul_mat(ops.QWeight.from_blocks(wtype, K, M, wq), torch.from_numpy(x).cuda()).cpu().numpy()
    out.append(float(np.abs(got - ref).max() / np.abs(ref).max()))
print(json.dumps({{"err": out, "status": int(_lib.lib().b200_kernel_status())}}))
"""


def run_child(cases, mode="1"):
    env = dict(os.environ, B200_MMQ_TC=mode)
    code = CHILD.format(here=HERE, root=ROOT, cases=cases)
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_tc_kernel_vs_oracle():
    """Full and ragged tiles: rows not a multiple of 128, columns not a multiple of 64, blocks not a multiple of 4,
    several column chunks, a split over K, and Q8_0 weights (mma.sync kernel on the canonical activation order)."""
    cases = [(2, 128, 128, 64), (2, 80, 512, 9), (2, 1000, 4096, 50), (2, 130, 160, 40), (2, 48, 14336, 20),
             (2, 300, 1024, 65), (2, 256, 256, 200), (8, 130, 160, 40), (8, 80, 512, 33)]
    res = run_child(cases)
    assert res["status"] == 0
    assert max(res["err"]) < 1e-3, res["err"]


CASES = [(2, 128, 128, 64), (2, 80, 512, 16), (2, 1000, 4096, 50), (2, 130, 160, 40), (2, 48, 14336, 20),
         (2, 300, 1024, 65), (2, 256, 256, 200), (2, 272, 2048 + 96, 128), (2, 4096, 4096, 64), (8, 130, 160, 40)]


def test_folded_scale_kernel_is_within_float_rounding_of_the_oracle():
    """Three product terms (B200_MMQ_TC=2): only the order of the fp32 sums differs from the reference, so the bound is
    twenty times tighter than the mul_mat tolerance (the tensor core's fp32 accumulation over
    14336 values measured 9e-6).  Both tile widths (up to 64 columns, more), ragged rows, columns
    and block counts, K splits; Q8_0 weights fall through to the mma.sync kernel."""
    res = run_child(CASES, "2")
    assert res["status"] == 0
    assert max(res["err"]) < 5e-5, res["err"]


def test_folded_scale_kernel_with_two_terms_is_within_the_mul_mat_tolerance():
    """Two product terms (B200_MMQ_TC=3): the weights are rounded to fp16 (2^-12 relative per term); that is inside the
    mul_mat tolerance of 1e-3, and visibly above the three-term error."""
    res = run_child(CASES, "3")
    assert res["status"] == 0
    assert max(res["err"]) < 1e-3, res["err"]

"""The stream-K work split of the tensor-core mul_mat kernel against the oracle.

By default the split is taken only where the cost model prefers it (wide products such as the stacked gate/up weight);
B200_MMQ_STREAMK=2 takes it wherever it is legal, which is read once per process, so the cases run in a child
interpreter.  Row groups here are cut into two or three parts; the sum must match the oracle and must not
depend on which CTA arrives last (two runs give identical bits).
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
from oracle.binding import Oracle
from cactus_b200 import ops, _lib
o = Oracle()
out = []
L = _lib.lib()
for (wtype, M, K, N) in {cases!r}:
    rng = np.random.default_rng(M + K + N)
    wq = o.quantize_weights(wtype, (rng.standard_normal((M, K)) * 0.02).astype(np.float32))
    x = rng.standard_normal((N, K)).astype(np.float32)
    ref, _ = o.mul_mat(wtype, wq, x)
    w = ops.QWeight.from_blocks(wtype, K, M, wq)
    xd = torch.from_numpy(x).cuda()
    n0 = L.b200_launch_count()
    got = ops.mul_mat(w, xd)
    launches = L.b200_launch_count() - n0
    again = ops.mul_mat(w, xd)
    out.append(dict(err=float(np.abs(got.cpu().numpy() - ref).max() / np.abs(ref).max()), same=bool(torch.equal(got, again)), launches=int(launches)))
print(json.dumps(out))
"""


def run_child(cases, mode):
    env = dict(os.environ, B200_MMQ_STREAMK=str(mode))
    code = CHILD.format(here=HERE, root=ROOT, cases=cases)
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


CASES = [(2, 28672, 4096, 64),    # the stacked gate/up weight of the 8B model: 224 row groups, heads and tails
         (2, 19200, 2048, 64),    # 150 row groups: heads of 10 block groups, tails shared by 146 CTAs
         (2, 38400, 1024, 50),    # 300 row groups over ~296 CTAs: the even deal, ragged columns
         (2, 19200, 2016, 40),    # K not a multiple of the 128-element block group
         (8, 19200, 2048, 33),    # Q8_0 weights
         (2, 4096, 4096, 64)]     # too few row groups: the cluster split, whatever the switch says

# narrower column classes (16- and 32-column CTAs hold more CTAs per SM, so the deals differ) and the output head
NARROW = [(2, 128256, 1024, 8), (2, 64000, 1024, 12), (2, 40064, 1024, 24), (2, 128256, 512, 3), (8, 51200, 512, 30)]


def test_streamk_forced_vs_oracle():
    res = run_child(CASES, 2)
    for c, r in zip(CASES, res):
        assert r["err"] < 1e-3, (c, r)
        assert r["same"], (c, r)
    # quantiser + counter reset + product: the split was really taken
    assert [r["launches"] for r in res[:4]] == [3, 3, 3, 3] and res[5]["launches"] == 2, res


def test_streamk_default_choice():
    """The cost model takes the split for the wide product and leaves the narrow one to the cluster split."""
    res = run_child([CASES[0], CASES[5]], 1)
    assert [r["launches"] for r in res] == [3, 2], res
    assert all(r["err"] < 1e-3 and r["same"] for r in res), res


@pytest.mark.parametrize("mode", [1, 2])
def test_streamk_narrow_column_classes(mode):
    res = run_child(NARROW, mode)
    for c, r in zip(NARROW, res):
        assert r["err"] < 1e-3 and r["same"], (c, r, mode)
    if mode == 2:
        assert any(r["launches"] == 3 for r in res), res

"""Why model-level comparisons cannot hold the per-op tolerances: the reference's own graph is discontinuous.

Every mul_mat re-quantises its input to int8 (quantize_row_q8_0, cactus/ggml-cpu/ggml-cpu-quants.c:732).  A float that
moves in its last bit can cross a rounding boundary, one int8 changes by 1, and that token's logits move by orders of
magnitude more than the float did.  This test shows it on the CPU oracle alone: the same small llama graph, run once as
is and once with every mul_mat output multiplied by 1 +- 2e-7 (less than two units in the last place), differs in its
logits by far more than 2e-7 -- and by no more than the bound the GPU model tests allow a kernel (3e-2 of the largest
logit).  A GPU kernel that sums the block products in another order than the AVX2 code perturbs its outputs by about
that much, so the model tests assert greedy-token equality and that bound, while the per-op tests stay strict."""
import numpy as np

from llama_ref import OracleLlama, tiny_model
from oracle.binding import Q4_0


class NoisyOracle:
    """The oracle with +-eps relative noise on what mul_mat returns; everything else passes through."""

    def __init__(self, oracle, eps, seed):
        self._o, self._eps, self._rng = oracle, eps, np.random.default_rng(seed)

    def __getattr__(self, name):
        return getattr(self._o, name)

    def mul_mat(self, wtype, wq, x, *a, **k):
        y, q8 = self._o.mul_mat(wtype, wq, x, *a, **k)
        sign = self._rng.integers(0, 2, y.shape).astype(np.float32) * 2 - 1
        return (y * (np.float32(1) + np.float32(self._eps) * sign)).astype(np.float32), q8


def run(o, cfg, arrays):
    from types import SimpleNamespace  # noqa: F401
    ref = OracleLlama(o, cfg, arrays, 256, acc_mode=1)
    rng = np.random.default_rng(1)
    lens = [9, 4, 14]
    tokens = rng.integers(0, cfg.vocab, sum(lens))
    pos = np.concatenate([np.arange(n) for n in lens])
    seq = np.concatenate([np.full(n, s) for s, n in enumerate(lens)])
    out = [ref.decode(tokens, pos, seq, np.arange(sum(lens)))]
    head = sum(lens)
    cur = out[0][np.cumsum(lens) - 1].argmax(-1)
    for step in range(3):
        out.append(ref.decode(cur, np.array(lens) + step, np.arange(3), head + np.arange(3)))
        head += 3
        cur = out[-1].argmax(-1)
    return np.concatenate(out)


def test_two_ulp_noise_on_mul_mat_outputs_moves_logits_by_orders_of_magnitude_more(oracle):
    from cactus_b200.engine import LlamaConfig
    cfg = LlamaConfig(n_layer=2, d_model=256, n_head=4, n_kv_head=2, d_ff=512, vocab=320, head_type=Q4_0)
    arrays = tiny_model(oracle, cfg)
    clean = run(oracle, cfg, arrays)
    eps = 2e-7
    worst = []
    for seed in range(3):
        noisy = run(NoisyOracle(oracle, eps, seed), cfg, arrays)
        rows = np.abs(noisy - clean).max(axis=1) / np.abs(clean).max()
        worst.append(rows.max())
        assert rows.max() < 3e-2, rows.max()          # the bound the GPU model tests use
    # a continuous graph would move by about eps; this one moves by at least a thousand times that on some token
    assert max(worst) > 1000 * eps, worst

"""Model level: a small llama (2 layers) run as ragged multi-sequence ubatches -- a prefill ubatch mixing
three sequences, then decode steps -- through the C-ABI engine, against the same graph composed from the
CPU oracle's ops.

Logits are compared in the normalised metric max|a-b|/max|b|: <= 1e-3 against the oracle graph whose
attention accumulates in double (same fp16-rounded Q, same f16 K/V), and <= 1e-3 plus the reference's own
distance from that graph against the oracle graph that accumulates the attention output in fp16 as the
reference does (cactus/ggml-cpu/ops.cpp:7103-7117) -- on this small model that fp16 accumulator alone
moves the logits by ~1e-2, far more than every other difference together.  Greedy tokens must be equal."""
import numpy as np
import pytest

from gpu_util import rel_max_err
from llama_ref import OracleLlama, tiny_model
from oracle.binding import Q4_0, Q8_0

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("head_type", [Q4_0, Q8_0])
@pytest.mark.parametrize("use_graphs", [False, True])
def test_ragged_prefill_then_decode(oracle, head_type, use_graphs):
    from cactus_b200.engine import LlamaConfig, LlamaEngine, LlamaWeights
    cfg = LlamaConfig(n_layer=2, d_model=256, n_head=4, n_kv_head=2, d_ff=512, vocab=320, head_type=head_type)
    arrays = tiny_model(oracle, cfg)
    n_cells = 256
    eng = LlamaEngine(LlamaWeights.from_numpy(cfg, arrays), n_cells, max_tokens=32, use_graphs=use_graphs)
    ref = OracleLlama(oracle, cfg, arrays, n_cells, acc_mode=1)
    ref16 = OracleLlama(oracle, cfg, arrays, n_cells, acc_mode=0)
    rng = np.random.default_rng(1)
    lens = [9, 4, 14]                          # three prompts in one ragged ubatch
    tokens = rng.integers(0, cfg.vocab, sum(lens))
    pos = np.concatenate([np.arange(n) for n in lens])
    seq = np.concatenate([np.full(n, s) for s, n in enumerate(lens)])
    slots = np.arange(sum(lens))
    got, ids = eng.decode(tokens, pos, seq, slots)
    want = ref.decode(tokens, pos, seq, slots)
    want16 = ref16.decode(tokens, pos, seq, slots)
    assert rel_max_err(got, want) < 1e-3
    assert rel_max_err(got, want16) < 1e-3 + rel_max_err(want16, want)
    last = np.cumsum(lens) - 1
    assert np.array_equal(ids[last], want[last].argmax(-1))
    head = sum(lens)
    cur = ids[last].copy()
    for step in range(3):                      # decode: one token per sequence, cells interleaved
        p = np.array(lens) + step
        s = np.arange(3)
        sl = head + np.arange(3)
        head += 3
        got, ids = eng.decode(cur, p, s, sl)
        want = ref.decode(cur, p, s, sl)
        want16 = ref16.decode(cur, p, s, sl)
        assert rel_max_err(got, want) < 1e-3, step
        assert rel_max_err(got, want16) < 1e-3 + rel_max_err(want16, want), step
        assert np.array_equal(ids, want.argmax(-1)), step
        cur = ids.copy()

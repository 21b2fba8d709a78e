"""One rank of the row-split tests (started by test_gpu_rowsplit.py with RANK / WORLD_SIZE / MASTER_* set).

Part 1: the join alone -- every rank pushes a known slice, placement must be exact, repeated to exercise the
collective counter.  Part 2: a small llama run row-split against the same model on one GPU (rank 0 holds both)."""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import numpy as np
import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo")
    from cactus_b200.engine import LlamaConfig, LlamaEngine, LlamaWeights
    from cactus_b200.rowsplit import RowSplit
    from llama_ref import tiny_model
    from oracle.binding import Oracle, Q4_0

    out = {"rank": rank}
    rs = RowSplit(rank, world, 64 << 20)
    # ---- part 1: the join ----
    T, M = 5, 64 * world
    Mg = M // world
    dst = rs.carve(8, M)
    st = torch.cuda.current_stream().cuda_stream
    ok = True
    for rep in range(3):
        src = (torch.arange(T * Mg, device="cuda", dtype=torch.float32).view(T, Mg) + 1000 * rank + 100000 * rep)
        rs.allgather(src, T, Mg, dst, st)
        torch.cuda.synchronize()
        want = torch.cat([torch.arange(T * Mg, dtype=torch.float32).view(T, Mg) + 1000 * r + 100000 * rep for r in range(world)], dim=1)
        ok = ok and bool(torch.equal(dst[:T].cpu(), want))
        dist.barrier()   # the next repetition overwrites dst: a one-buffer test needs what the model's buffer rotation gives
    out["join_exact"] = ok
    out["join_status"] = rs.status()
    # ---- part 1b: a stacked product -- this rank's rows of two weights in one mul_mat, each piece at its own columns ----
    oracle = Oracle()
    from cactus_b200 import ops
    from cactus_b200.ops import QWeight
    from cactus_b200._lib import lib
    rngw = np.random.default_rng(7)
    K, Ma, Mb = 256, 64 * world, 32 * world
    wa = QWeight.from_blocks(Q4_0, K, Ma, oracle.quantize_weights(Q4_0, (rngw.standard_normal((Ma, K)) * 0.05).astype(np.float32)))
    wb = QWeight.from_blocks(Q4_0, K, Mb, oracle.quantize_weights(Q4_0, (rngw.standard_normal((Mb, K)) * 0.05).astype(np.float32)))
    sa, sb = wa.row_slice(rank * Ma // world, (rank + 1) * Ma // world), wb.row_slice(rank * Mb // world, (rank + 1) * Mb // world)
    stacked = QWeight.cat([sa, sb])
    stacked.parts = [(sa.M, sa.row0), (sb.M, Ma + sb.row0)]
    joined = rs.carve(8, Ma + Mb)
    ws = torch.empty(max(256, lib().b200_mul_mat_workspace_bytes(Q4_0, K, stacked.M, 8)), dtype=torch.uint8, device="cuda")
    stacked_err = 0.0
    for N in (1, 5):
        x = torch.from_numpy(rngw.standard_normal((N, K)).astype(np.float32)).cuda()
        act = torch.empty(lib().b200_act_bytes(K, N), dtype=torch.uint8, device="cuda")
        from cactus_b200._lib import check
        check(lib().b200_quantize_activations(x.data_ptr(), K * 4, K, N, act.data_ptr(), act.numel(), 0, st))
        rs.mul_mat(stacked, act, N, joined, ws, st)
        torch.cuda.synchronize()
        want = torch.cat([ops.mul_mat(wa, x), ops.mul_mat(wb, x)], dim=1)
        stacked_err = max(stacked_err, float((joined[:N] - want).abs().max() / want.abs().max()))
        dist.barrier()
    out["stacked_err"] = stacked_err
    # ---- part 2: the model ----
    cfg = LlamaConfig(n_layer=2, d_model=256, n_head=4, n_kv_head=2, d_ff=512, vocab=320, head_type=Q4_0)
    arrays = tiny_model(oracle, cfg)
    full = LlamaWeights.from_numpy(cfg, arrays)
    eng = LlamaEngine(full.shard(rank, world), 256, max_tokens=32, use_graphs=True, split=rs)
    rng = np.random.default_rng(1)
    lens = [9, 4, 14]
    tokens = rng.integers(0, cfg.vocab, sum(lens))
    pos = np.concatenate([np.arange(n) for n in lens])
    seq = np.concatenate([np.full(n, s) for s, n in enumerate(lens)])
    slots = np.arange(sum(lens))
    steps = [(tokens, pos, seq, slots)]
    for step in range(2):
        steps.append((rng.integers(0, cfg.vocab, 3), np.array(lens) + step, np.arange(3), sum(lens) + 3 * step + np.arange(3)))
    got = [eng.decode(*s)[0].copy() for s in steps for _ in range(1)]
    # the same with attention replicated on every rank (what the engine does when the head counts do not divide)
    eng2 = LlamaEngine(full.shard(rank, world), 256, max_tokens=32, use_graphs=False, split=rs, head_parallel=False)
    got2 = [eng2.decode(*s)[0].copy() for s in steps]
    out["head_parallel"] = bool(eng.hp) and not eng2.hp
    out["replicated_attention_err"] = max(float(np.abs(a - b).max() / np.abs(b).max()) for a, b in zip(got2, got))
    out["model_status"] = rs.status()
    sums = torch.tensor([float(np.abs(g).sum()) for g in got], dtype=torch.float64)
    gathered = [torch.zeros_like(sums) for _ in range(world)]
    dist.all_gather(gathered, sums)
    out["ranks_agree"] = all(bool(torch.equal(gathered[0], t)) for t in gathered)   # every rank ends with the same logits
    if rank == 0:
        single = LlamaEngine(full, 256, max_tokens=32, use_graphs=False)
        errs, same_argmax = [], True
        for s, g in zip(steps, got):
            want, _ = single.decode(*s)
            errs.append(float(np.abs(g - want).max() / np.abs(want).max()))
            same_argmax = same_argmax and bool(np.array_equal(g.argmax(-1), want.argmax(-1)))
        out["max_err_vs_single_gpu"] = max(errs)
        out["same_argmax"] = same_argmax
    dist.barrier()
    rs.close()
    print("RESULT " + json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""The N > 1 plumbing of the benchmark on CPU: two gloo ranks, the job time is the slowest rank's, the job
throughput sums the replicas."""
import os
import socket

import torch.multiprocessing as mp


def _worker(rank, world, port, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from cactus_b200 import dist as d
    r, w = d.init("gloo")
    assert (r, w) == (rank, world)
    d.barrier()
    seconds = 2.0 if rank == 0 else 3.0          # rank 1 is slower
    out[rank] = (d.max_over_ranks(seconds), d.job_throughput(64 * 10, seconds))
    d.shutdown()


def test_two_rank_timing_reduction():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    for rank in (0, 1):
        t, thr = out[rank]
        assert t == 3.0
        assert abs(thr - 2 * 640 / 3.0) < 1e-9


def test_single_process_is_identity():
    from cactus_b200 import dist as d
    assert d.max_over_ranks(1.5) == 1.5
    assert d.job_throughput(64, 2.0) == 32.0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rowsplit_worker(rank, world, port, q):
    """Host logic of the row split on CPU ranks: every rank slices its rows out of the block stream, computes its part
    of the product with the oracle, and the parts joined in rank order are the full product, bit for bit."""
    import sys
    import numpy as np
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cactus_b200.rowsplit import row_bounds, slice_blocks
    from oracle.binding import Oracle, Q4_0
    o = Oracle()
    M, K, N = 96, 256, 5
    rng = np.random.default_rng(7)
    wq = o.quantize_weights(Q4_0, (rng.standard_normal((M, K)) * 0.02).astype(np.float32))
    x = rng.standard_normal((N, K)).astype(np.float32)
    full, _ = o.mul_mat(Q4_0, wq, x)
    b = row_bounds(M, world)
    part, _ = o.mul_mat(Q4_0, slice_blocks(np.asarray(wq), M, rank, world), x)
    assert part.shape == (N, b[rank + 1] - b[rank])
    parts = [torch.zeros((N, b[r + 1] - b[r])) for r in range(world)]
    dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(part)))
    joined = torch.cat(parts, dim=1).numpy()
    q.put((rank, bool(np.array_equal(joined, full)), b))
    dist.destroy_process_group()


def test_rowsplit_host_logic_gloo():
    from cactus_b200.rowsplit import row_bounds
    import pytest as _pytest
    assert row_bounds(128256, 8) == [16032 * r for r in range(8)] + [128256]
    assert row_bounds(80, 1) == [0, 80]
    with _pytest.raises(Exception):
        row_bounds(48, 2)   # 3 tiles do not split over 2 ranks
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_rowsplit_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = [q.get(timeout=120) for _ in ps]
    for p in ps:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in got)
    assert all(b == [0, 48, 96] for _, _, b in got)

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

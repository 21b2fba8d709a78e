"""Multi-GPU plumbing of the benchmark: one process per GPU, each running its own replica (own weights, own 64
sequences).  The path has no data-path collective -- the 8B model fits one GPU -- so the only exchange is the
timing reduction: every rank contributes its device-measured time, the job time is the maximum, and the job's
throughput is the sum of the replicas' work over that time."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def env_rank():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def init(backend: str, device=None):
    rank, world, _ = env_rank()
    if world > 1 and not dist.is_initialized():
        kw = {"device_id": device} if (backend == "nccl" and device is not None) else {}
        dist.init_process_group(backend, **kw)
    return rank, world


def barrier():
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def max_over_ranks(value: float, device="cpu") -> float:
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def job_throughput(units_per_rank: float, seconds_this_rank: float, device="cpu") -> float:
    """Whole-job units per second: all ranks' units over the slowest rank's time."""
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    return world * units_per_rank / max_over_ranks(seconds_this_rank, device)


def shutdown():
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()

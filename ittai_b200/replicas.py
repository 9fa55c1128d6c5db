"""Replica aggregation for multi-GPU runs: the Qwen3-0.6B and SigLIP paths do not shard (the model is 1.2 GB), so N GPUs
run N independent streams.  The only cross-rank step is timing: a barrier on both sides of the timed region, the
maximum duration over ranks, and the sum of the units the ranks processed.  The reference has no multi-GPU code."""
from __future__ import annotations

import torch
import torch.distributed as dist


def barrier(device=None) -> None:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    if device is not None and torch.device(device).type == "cuda":
        torch.cuda.synchronize(device)


def aggregate(durations_ms, units: float, device="cpu"):
    """``durations_ms``: this rank's timed durations (one per metric); ``units``: work this rank did in the primary one.

    Returns (max over ranks of each duration, sum over ranks of units).  No data-path collective: two tiny reductions."""
    t = torch.tensor(list(durations_ms), dtype=torch.float64, device=device)
    u = torch.tensor([float(units)], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(u, op=dist.ReduceOp.SUM)
    return t.tolist(), float(u.item())

"""Multi-GPU operation: independent replicas, one process per GPU, no data-path collective.

A pi0 request is a serial chain of ~1 800 dependent stages at batch 1, so it is not sharded: request ``i``
goes to replica ``i mod world`` and every replica holds the full NVFP4 weight set.  ``torch.distributed`` is
used only as plumbing around the measurement: a barrier before and after the timed region and a reduction of
each replica's statistics (MAX for latencies, SUM for throughput).  Works with the ``nccl`` backend on GPUs and
with ``gloo`` on CPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def requests_for(rank: int, world: int, total: int):
    """Indices of the requests replica ``rank`` serves (round robin)."""
    if world < 1 or not 0 <= rank < world or total < 0:
        raise ValueError("invalid replica geometry")
    return list(range(rank, total, world))


def reduce_stats(latencies_ms, actions_per_request: int, device="cpu"):
    """Combine per-replica latency samples: returns dict(p50_ms=max over replicas, p90_ms=max,
    actions_per_s=sum over replicas of actions_per_request / p50)."""
    s = sorted(float(v) for v in latencies_ms)
    if not s:
        raise ValueError("no samples")

    def pct(q):
        pos = (len(s) - 1) * q
        lo, hi = int(pos), min(int(pos) + 1, len(s) - 1)
        return s[lo] + (s[hi] - s[lo]) * (pos - lo)

    p50, p90 = pct(0.5), pct(0.9)
    worst = torch.tensor([p50, p90], dtype=torch.float64, device=device)
    rate = torch.tensor([actions_per_request * 1e3 / p50], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        dist.all_reduce(rate, op=dist.ReduceOp.SUM)
    return {"p50_ms": float(worst[0]), "p90_ms": float(worst[1]), "actions_per_s": float(rate[0])}

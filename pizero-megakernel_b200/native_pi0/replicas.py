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


# ---------------------------------------------------------------------------------------------------------------
# A pool of replicas behind one submit() call: one worker process per GPU, each with its own engine and policy.
def _replica_worker(index, device, factory, requests, results):
    """Worker process: build the policy on `device`, then serve observations until a None arrives."""
    try:
        policy = factory(device)
        results.put((index, None, "ready"))
        while True:
            item = requests.get()
            if item is None:
                break
            ticket, observation, noise = item
            try:
                results.put((index, ticket, policy.infer(observation, noise)))
            except Exception as error:                      # the request fails, the replica stays up
                results.put((index, ticket, error))
    except Exception as error:
        results.put((index, None, error))


class ReplicaPool:
    """Independent pi0 replicas, one process per device, requests dealt round robin (request i -> replica i mod n) and
    answered in submission order.  ``factory(device) -> policy`` runs inside each worker (it builds the engine there);
    with CUDA devices use the ``spawn`` start method and a module-level factory.  No replica ever talks to another."""

    def __init__(self, factory, devices, *, start_method="spawn", startup_timeout=600.0):
        import multiprocessing
        ctx = multiprocessing.get_context(start_method)
        self.devices = list(devices)
        if not self.devices:
            raise ValueError("at least one device")
        self.results = ctx.Queue()
        self.requests = [ctx.Queue() for _ in self.devices]
        self.workers = [ctx.Process(target=_replica_worker, args=(i, d, factory, self.requests[i], self.results), daemon=True)
                        for i, d in enumerate(self.devices)]
        for w in self.workers:
            w.start()
        self.submitted = 0
        self._done = {}
        for _ in self.workers:
            index, _, message = self.results.get(timeout=startup_timeout)
            if isinstance(message, Exception):
                self.close()
                raise RuntimeError(f"replica {index} failed to start: {message!r}")

    def submit(self, observation, noise=None):
        """Queue one observation; returns its ticket (the submission index)."""
        ticket = self.submitted
        self.requests[requests_for_ticket(ticket, len(self.devices))].put((ticket, observation, noise))
        self.submitted += 1
        return ticket

    def result(self, ticket, timeout=120.0):
        while ticket not in self._done:
            _, t, value = self.results.get(timeout=timeout)
            self._done[t] = value
        value = self._done.pop(ticket)
        if isinstance(value, Exception):
            raise RuntimeError(f"request {ticket} failed: {value!r}")
        return value

    def map(self, observations):
        tickets = [self.submit(o) for o in observations]
        return [self.result(t) for t in tickets]

    def close(self):
        for q in self.requests:
            q.put(None)
        for w in self.workers:
            w.join(timeout=30)
            if w.is_alive():
                w.terminate()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()


def requests_for_ticket(ticket: int, world: int) -> int:
    """Replica that serves submission number `ticket` (the inverse view of ``requests_for``)."""
    return ticket % world

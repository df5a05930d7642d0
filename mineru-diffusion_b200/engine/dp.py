"""Request-level data parallelism: one engine replica per GPU, no data-path
collective (requests share nothing: prefix-cache hashing is off in the
reference, ``engines/nano_dvlm/nanovllm/engine/block_manager.py:65-66``).

``partition_requests`` assigns requests to ranks; ``reduce_throughput``
combines per-rank results the way the benchmark reports them (tokens summed,
time = slowest rank).
"""
from __future__ import annotations

import heapq

import torch
import torch.distributed as dist


def _longest_first(costs: list[float], world_size: int) -> list[list[int]]:
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    heap = [(0, r) for r in range(world_size)]
    heapq.heapify(heap)
    out: list[list[int]] = [[] for _ in range(world_size)]
    for i in order:
        load, r = heapq.heappop(heap)
        out[r].append(i)
        heapq.heappush(heap, (load + costs[i], r))
    return out


def partition_requests(costs: list[float], world_size: int, steps: list[int] | None = None,
                       step_cost: float = 0.0) -> list[list[int]]:
    """Greedy longest-first bin packing of request indices; deterministic, so every rank computes the same split.

    With ``costs`` alone (prompt + output tokens, or any additive estimate) a rank's load is the sum of its
    requests' costs.  A replica, however, steps until its *last* request is done, and every step has a fixed
    part (the weights are streamed whatever the batch): with ``steps`` (how many engine steps request i stays in
    flight) and ``step_cost`` (that fixed part, in the unit of ``costs``) the load of a rank is
    ``sum(costs) + step_cost * max(steps)`` over its requests, and each request goes to the rank whose load ends
    lowest -- long-running requests gather on few ranks instead of setting the step count of all of them.  The
    split returned is never worse under that model than the one the additive costs alone would give."""
    if world_size < 1:
        raise ValueError("world_size must be positive")
    if steps is not None and len(steps) != len(costs):
        raise ValueError("steps must have one entry per request")
    out = _longest_first(costs, world_size)
    if steps is not None and step_cost > 0:
        order = sorted(range(len(costs)), key=lambda i: (-(costs[i] + step_cost * steps[i]), i))
        aware: list[list[int]] = [[] for _ in range(world_size)]
        total = [0.0] * world_size
        longest = [0] * world_size
        for i in order:
            best = min(range(world_size),
                       key=lambda r: (total[r] + costs[i] + step_cost * max(longest[r], steps[i]), total[r], r))
            aware[best].append(i)
            total[best] += costs[i]
            longest[best] = max(longest[best], steps[i])
        worst = lambda parts: max(modelled_load(p, costs, steps, step_cost) for p in parts)   # noqa: E731
        if worst(aware) < worst(out):
            out = aware
    for part in out:
        part.sort()
    return out


def modelled_load(part: list[int], costs: list[float], steps: list[int] | None = None, step_cost: float = 0.0) -> float:
    """Load of one rank under the model ``partition_requests`` balances."""
    if not part:
        return 0.0
    load = float(sum(costs[i] for i in part))
    if steps is not None and step_cost > 0:
        load += step_cost * max(steps[i] for i in part)
    return load


def reduce_throughput(tokens: int, times_ms: list[float], counters: list[int], device) -> tuple[int, list[float], list[int]]:
    """Whole-job totals over the process group: tokens and counters summed,
    each time the maximum over ranks.  A single process returns its inputs."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return tokens, list(times_ms), list(counters)
    t = torch.tensor(times_ms, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    c = torch.tensor([tokens, *counters], dtype=torch.int64, device=device)
    dist.all_reduce(c, op=dist.ReduceOp.SUM)
    c = c.tolist()
    return int(c[0]), t.tolist(), [int(x) for x in c[1:]]

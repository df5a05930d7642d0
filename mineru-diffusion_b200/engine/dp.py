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


def partition_requests(costs: list[int], world_size: int) -> list[list[int]]:
    """Greedy longest-first bin packing of request indices by cost (prompt +
    output tokens); deterministic, so every rank computes the same split."""
    if world_size < 1:
        raise ValueError("world_size must be positive")
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    heap = [(0, r) for r in range(world_size)]
    heapq.heapify(heap)
    out: list[list[int]] = [[] for _ in range(world_size)]
    for i in order:
        load, r = heapq.heappop(heap)
        out[r].append(i)
        heapq.heappush(heap, (load + costs[i], r))
    for part in out:
        part.sort()
    return out


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

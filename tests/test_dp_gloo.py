"""Request-parallel bookkeeping on CPU ranks (gloo, world size 2)."""
import importlib
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    dp = importlib.import_module("mineru-diffusion_b200.engine.dp")
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", world_size=world, rank=rank)
    costs = [900, 100, 500, 450, 50, 700, 300, 20]
    parts = dp.partition_requests(costs, world)
    mine = parts[rank]
    tokens = sum(costs[i] for i in mine)
    total, (t_max, t2), (launches,) = dp.reduce_throughput(tokens, [10.0 + rank, 5.0 - rank], [100 * (rank + 1)], "cpu")
    torch.save(dict(parts=parts, total=total, t_max=t_max, t2=t2, launches=launches), os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_partition_is_balanced_and_complete(mdb):
    dp = importlib.import_module("mineru-diffusion_b200.engine.dp")
    g = torch.Generator().manual_seed(5)
    costs = (torch.randint(512, 8193, (512,), generator=g) + torch.randint(512, 8193, (512,), generator=g)).tolist()
    for world in (1, 2, 4, 8):
        parts = dp.partition_requests(costs, world)
        assert sorted(i for p in parts for i in p) == list(range(512))
        loads = [sum(costs[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(costs)
        assert max(loads) <= 1.01 * sum(costs) / world + max(costs) / world
    assert dp.partition_requests([], 2) == [[], []]


def test_partition_with_step_term_gathers_long_requests(mdb):
    """A replica steps until its last request is done and every step has a fixed cost: with that term in the
    load the partitioner must not let one long request set the step count of every rank."""
    dp = importlib.import_module("mineru-diffusion_b200.engine.dp")
    g = torch.Generator().manual_seed(9)
    for world in (2, 4, 8):
        n = 32
        steps = torch.randint(6, 49, (n,), generator=g).tolist()
        costs = [float(300 * s + int(torch.randint(2000, 33000, (1,), generator=g))) for s in steps]
        step_cost = 1600.0
        plain = dp.partition_requests(costs, world)
        aware = dp.partition_requests(costs, world, steps=steps, step_cost=step_cost)
        assert sorted(i for p in aware for i in p) == list(range(n))
        assert aware == dp.partition_requests(costs, world, steps=steps, step_cost=step_cost)   # deterministic
        worst = lambda parts: max(dp.modelled_load(p, costs, steps, step_cost) for p in parts)  # noqa: E731
        assert worst(aware) <= worst(plain) + 1e-6, (world, worst(aware), worst(plain))
    # without the step term the split is the plain longest-first one
    assert dp.partition_requests(costs, 4, steps=steps, step_cost=0.0) == dp.partition_requests(costs, 4)


def test_reduce_throughput_two_ranks(tmp_path):
    port = 29600 + os.getpid() % 200
    mp.start_processes(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    r0, r1 = torch.load(tmp_path / "r0.pt"), torch.load(tmp_path / "r1.pt")
    assert r0 == r1                                   # every rank sees the same totals
    assert r0["total"] == 900 + 100 + 500 + 450 + 50 + 700 + 300 + 20
    assert r0["t_max"] == 11.0 and r0["t2"] == 5.0    # slowest rank wins each time
    assert r0["launches"] == 300
    assert sorted(i for p in r0["parts"] for i in p) == list(range(8))


def test_reduce_throughput_single_process():
    dp = importlib.import_module("mineru-diffusion_b200.engine.dp")
    assert dp.reduce_throughput(7, [1.5], [3], "cpu") == (7, [1.5], [3])

"""World-size-2 checks of the benchmark's multi-rank logic on CPU (gloo): sharding plan and max-over-ranks timing."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import bench
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        weak = bench.workload("c2")
        strong = bench.workload("c5")
        res = {
            "weak": bench.shard_of(weak, world, rank),
            "strong": bench.shard_of(strong, world, rank),
            "max": bench.max_over_ranks(10.0 + 5 * rank, world, torch.device("cpu")),
        }
        out.put((rank, res))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_and_reduce():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(out.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    # weak scaling: every rank a whole 32-head batch, two batches in the job
    assert got[0]["weak"] == (32, 0, 2) and got[1]["weak"] == (32, 0, 2)
    # strong scaling: 64 heads cut into contiguous halves that cover every head once
    assert got[0]["strong"] == (32, 0, 1) and got[1]["strong"] == (32, 32, 1)
    # the job's time is the slowest rank's, on every rank
    assert got[0]["max"] == 15.0 and got[1]["max"] == 15.0


def test_workload_definitions_match_the_benchmark_configs():
    sys.path.insert(0, ROOT)
    import bench
    c2 = bench.workload("c2")
    assert c2["lengths"] == [2943, 3503, 2192, 1807, 3696, 649, 1594] and bench.pairs(c2["lengths"]) == 22804220
    c5 = bench.workload("c5")
    assert len(c5["lengths"]) == 70 and sum(c5["lengths"]) == 131072 and max(c5["lengths"]) == 16384
    assert bench.pairs(c5["lengths"]) == 415383762
    assert abs(bench.flops_fwd_bwd(32, 128, c2["lengths"]) - 1.308e12) < 1e9

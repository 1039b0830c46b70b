"""The multi-GPU path is independent replicas with no data-path collective; what the ranks share is
the timing reduction of bench.py (barrier, max over ranks, whole-job throughput) and the rule that
each rank draws its own episode. Exercised here with two `gloo` ranks on the CPU."""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank: int, world: int, port: int, out):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import bench
    from flash_vla_b200.synthetic import bench_inputs
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        assert bench.dist_env() == (rank, rank, world)
        bench.barrier(world)
        local_ms = 100.0 + 50.0 * rank                      # rank 1 is the slow replica
        slowest = bench.max_over_ranks(local_ms, world)
        images, _, noise = bench_inputs(seed=rank)
        out.put((rank, slowest, bench.job_throughput(world, 10, slowest), float(noise.sum()), float(images.mean())))
    finally:
        dist.destroy_process_group()


def test_two_rank_timing_reduction_and_distinct_episodes():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, slow0, thr0, n0, _), (r1, slow1, thr1, n1, _) = results
    assert (r0, r1) == (0, 1)
    assert slow0 == slow1 == 150.0                           # max over ranks, identical on every rank
    assert abs(thr0 - 2 * 10 / 0.150) < 1e-9 and thr0 == thr1
    assert n0 != n1                                          # each replica works on its own episode


def test_single_rank_paths_need_no_process_group():
    sys.path.insert(0, str(ROOT))
    import bench
    assert bench.max_over_ranks(12.5, 1) == 12.5
    assert bench.job_throughput(1, 30, 300.0) == 100.0
    cfg = bench.workload_config(4)
    assert cfg["replicas"] == 4 and "no collective" in cfg["parallelism"]

"""The N > 1 bookkeeping of bench.py on two gloo ranks (CPU): the job's time is the slowest rank's,
the job's throughput counts every rank's tokens, and only rank 0 reports."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import bench

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = 10.0 + 5.0 * rank  # rank 1 is slower
        dist.barrier()
        slowest = bench.max_over_ranks(mine, dist, torch.device("cpu"))
        value = bench.job_throughput(world, bench.step_flops(), 4, slowest)
        out.put((rank, slowest, value))
    finally:
        dist.destroy_process_group()


def test_two_rank_timing_and_aggregate():
    import bench

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, slowest, value in results:
        assert slowest == pytest.approx(15.0)
        assert value == pytest.approx(2 * bench.step_flops() * 4 / 15e-3 / 1e12)
    # single rank: no collective at all
    assert bench.max_over_ranks(7.0, None, torch.device("cpu")) == 7.0
    assert bench.step_flops() == pytest.approx(7.306e12, rel=1e-3)

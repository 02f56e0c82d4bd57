"""Host-side logic of the N > 1 benchmark path on CPU: two gloo ranks."""
import os
import sys
from pathlib import Path

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    import bench
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # rank 1 is the slow replica: the job's time is the maximum over ranks, tokens add up
    dev_ms, wall_s = (100.0, 0.11) if rank == 0 else (160.0, 0.17)
    agg = bench.aggregate_over_ranks(dev_ms, wall_s, 512, world, dist)
    dist.barrier()
    out[rank] = agg
    dist.destroy_process_group()


def test_replica_aggregation_two_gloo_ranks():
    world = 2
    port = 29000 + os.getpid() % 2000
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    for rank in range(world):
        agg = out[rank]
        assert agg["tokens"] == 1024
        assert agg["dev_ms"] == pytest.approx(160.0) and agg["wall_s"] == pytest.approx(0.17)
        assert agg["value"] == pytest.approx(1024 / 0.160)
        assert agg["e2e"] == pytest.approx(1024 / 0.17)


def test_single_rank_aggregation_needs_no_process_group():
    sys.path.insert(0, str(ROOT))
    import bench
    agg = bench.aggregate_over_ranks(50.0, 0.06, 256, 1)
    assert agg["value"] == pytest.approx(5120.0) and agg["e2e"] == pytest.approx(256 / 0.06)


def test_bench_env_parsing(monkeypatch):
    sys.path.insert(0, str(ROOT))
    import bench
    monkeypatch.setenv("RANK", "3")
    monkeypatch.setenv("WORLD_SIZE", "8")
    monkeypatch.setenv("LOCAL_RANK", "3")
    assert bench.dist_env() == (3, 8, 3)

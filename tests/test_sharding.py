"""The multi-GPU plan on CPU ranks: (batch, head) problems split over ranks with no exchange on
the data path, one gather at the end, and times reduced as the max over ranks. Runs two gloo
processes; the attention values come from the CPU oracle here (the checker), since the point
is the partition and the gather, not the kernels."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT))
    import bench
    from oracle import sdpa_oracle as oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bench.WORKLOADS["tiny"] = (2, 3, 64, 32, True, True, 1.0, "normal", 11, "test workload")
        first, count = bench.shard_range(6, rank, world)
        q, k, v, do = bench.shard_inputs("tiny", first, count, True)
        out, lse = oracle.sdpa_forward(q, k, v, causal=True, scale=32**-0.5)
        mine = torch.from_numpy(out.view(np.int16).copy())
        whole = torch.empty((6, 64, 32), dtype=torch.int16)
        dist.all_gather_into_tensor(whole.view(torch.uint8), mine.view(torch.uint8))  # bytes: gloo has no 16-bit integer type
        slowest = bench.reduce_max(float(rank + 1), dist, torch.device("cpu"))
        if rank == 0:
            np.save(Path(out_dir) / "whole.npy", whole.numpy())
            np.save(Path(out_dir) / "slowest.npy", np.array([slowest]))
    finally:
        dist.destroy_process_group()


def test_two_ranks_partition_and_gather(tmp_path):
    import torch.multiprocessing as mp

    import bench
    from conftest import BF16
    from oracle import sdpa_oracle as oracle

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    whole = np.load(tmp_path / "whole.npy").view(BF16)
    bench.WORKLOADS["tiny"] = (2, 3, 64, 32, True, True, 1.0, "normal", 11, "test workload")
    q, k, v, _ = bench.shard_inputs("tiny", 0, 6, True)  # the unsharded job
    want, _ = oracle.sdpa_forward(q, k, v, causal=True, scale=32**-0.5)
    np.testing.assert_array_equal(whole.view(np.uint16), want.view(np.uint16))
    assert np.load(tmp_path / "slowest.npy")[0] == 2.0


def test_shard_ranges_cover_every_problem_once():
    import bench

    for bh, world in ((256, 1), (256, 2), (256, 4), (256, 8), (160, 8)):
        seen = []
        for rank in range(world):
            first, count = bench.shard_range(bh, rank, world)
            seen += list(range(first, first + count))
        assert seen == list(range(bh))
    with pytest.raises(ValueError, match="do not split evenly"):
        bench.shard_range(10, 0, 4)


def test_inputs_do_not_depend_on_the_sharding():
    import bench

    bench.WORKLOADS["tiny"] = (2, 3, 64, 32, True, True, 1.0, "normal", 11, "test workload")
    whole = bench.shard_inputs("tiny", 0, 6, True)
    for first, count in ((0, 3), (3, 3), (4, 2)):
        part = bench.shard_inputs("tiny", first, count, True)
        for a, b in zip(whole, part):
            np.testing.assert_array_equal(a[first : first + count].view(np.uint16), b.view(np.uint16))

"""CPU: the host logic of the multi-GPU path (request sharding, max-over-ranks timing, result gather),
single-process properties plus a world_size-2 run over the gloo backend."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from turbotransformers_b200 import sharding, synthetic


def test_contiguous_shards_partition():
    for n, w in [(256, 8), (256, 4), (64, 2), (7, 4), (1, 2)]:
        s = sharding.contiguous_shards(n, w)
        assert sorted(i for part in s for i in part) == list(range(n)) and len(s) == w
    assert [len(p) for p in sharding.contiguous_shards(256, 8)] == [32] * 8


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_balanced_shards_partition_and_balance(world):
    lens = synthetic.varlen_lengths(64, 8, 512, 0)
    s = sharding.balanced_shards(lens, world)
    assert sorted(i for part in s for i in part) == list(range(64))
    assert sharding.imbalance(lens, s) < 1.05
    naive = sharding.contiguous_shards(64, world)
    assert sharding.imbalance(lens, s) <= sharding.imbalance(lens, naive) + 1e-9


def test_job_throughput_uses_slowest_rank():
    assert sharding.job_throughput([64, 64], [5.0, 10.0]) == pytest.approx(12800.0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lens = synthetic.varlen_lengths(16, 8, 64, 3)
        shards = sharding.balanced_shards(lens, world)
        # each rank "computes" a row per request: the request index and its length
        local = torch.tensor([[float(i), float(lens[i])] for i in shards[rank]])
        gathered = sharding.gather_rows(local, shards, rank)
        ms = sharding.reduce_max_ms(3.0 + rank)  # rank 1 is slower
        dist.barrier()
        if rank == 0:
            torch.save({"gathered": gathered, "ms": ms, "lens": lens}, out)
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_gloo(tmp_path):
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    r = torch.load(out)
    assert r["ms"] == 4.0  # the max over ranks
    assert r["gathered"][:, 0].tolist() == [float(i) for i in range(16)]  # request order restored
    assert r["gathered"][:, 1].tolist() == [float(n) for n in r["lens"]]

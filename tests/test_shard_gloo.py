"""The N>1 host path on CPU: two gloo ranks shard a batch, agree on a max-over-ranks timing and on
the aggregate, with no collective on the data path."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tracea_b200 import shard


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_images, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a, b = shard.shard_range(n_images, rank, world)
        # each rank "processes" its own images; pretend rank r took (r + 1) ms
        elapsed = shard.max_over_ranks(float(rank + 1))
        total = shard.sum_over_ranks(float(b - a))
        dist.barrier()
        torch.save({"range": (a, b), "elapsed": elapsed, "total": total}, os.path.join(out_dir, "r%d.pt" % rank))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_images", [256, 7])
def test_two_ranks_shard_and_reduce(tmp_path, n_images):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), n_images, str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(os.path.join(str(tmp_path), "r%d.pt" % r)) for r in range(world)]
    assert res[0]["range"][0] == 0 and res[0]["range"][1] == res[1]["range"][0] and res[1]["range"][1] == n_images
    for r in res:
        assert r["elapsed"] == 2.0       # the slowest rank sets the step time
        assert r["total"] == float(n_images)


def test_max_over_ranks_without_a_process_group():
    assert shard.max_over_ranks(3.5) == 3.5

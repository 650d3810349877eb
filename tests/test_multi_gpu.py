"""The N > 1 path on CPU: two gloo ranks shard a frame stream, time their part and aggregate as bench.py does."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from visualmesh_b200 import sharding
from visualmesh_b200 import workloads as W


def test_shards_are_disjoint_and_cover_everything():
    for n in (0, 1, 7, 64, 4096):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                b, e = sharding.shard_bounds(n, r, world)
                assert 0 <= b <= e <= n
                seen += list(range(b, e))
            assert seen == list(range(n))
            sizes = [len(sharding.shard(list(range(n)), r, world)) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
            rr = sorted(sum((sharding.round_robin(list(range(n)), r, world) for r in range(world)), []))
            assert rr == list(range(n))
    with pytest.raises(ValueError):
        sharding.shard_bounds(4, 2, 2)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    wl = W.config(4, seed=3, n_frames=10)  # the height-mixed stream
    mine = sharding.round_robin(wl.frames, rank, world)
    # every rank sees the same seeded stream and takes its own frames of it
    heights = [fr.mesh.h for fr in mine]
    points = sum(int(1000 * h) for h in heights)
    dist.barrier()
    # the aggregation bench.py runs around its timed regions: slowest rank's time, whole-job counts
    elapsed = sharding.max_over_ranks(dist, 0.5 + rank)
    frames = int(sharding.sum_over_ranks(dist, len(mine)))
    pts = int(sharding.sum_over_ranks(dist, points))
    out[rank] = (elapsed, frames, pts, len(mine), [fr.image_seed for fr in mine])
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_aggregate():
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    wl = W.config(4, seed=3, n_frames=10)
    assert out[0][:3] == out[1][:3]
    elapsed, frames, pts = out[0][:3]
    assert elapsed == 1.5              # the slowest rank sets the time
    assert frames == 10                # whole-job frames, not per rank
    assert pts == sum(int(1000 * fr.mesh.h) for fr in wl.frames)
    assert sorted(out[0][4] + out[1][4]) == sorted(fr.image_seed for fr in wl.frames)
    assert not set(out[0][4]) & set(out[1][4])
    # frame i goes to rank i mod world, as configuration 4's stream is dealt over the GPUs
    assert out[0][4] == [fr.image_seed for fr in wl.frames[0::2]] and out[1][4] == [fr.image_seed for fr in wl.frames[1::2]]


def test_aggregation_without_a_process_group_is_the_identity():
    assert sharding.max_over_ranks(None, 1.25) == 1.25
    assert sharding.sum_over_ranks(None, 7) == 7.0

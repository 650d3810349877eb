"""Frame-level data parallelism: frames are independent, so a stream is dealt out to the GPUs of a box and nothing is
exchanged on the data path. The only communication is the bookkeeping around a timed run (a barrier, the maximum of the
per-rank durations, the sum of the per-rank counts), which works on any torch.distributed backend."""
from typing import List, Sequence, Tuple


def shard_bounds(n_items: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous shard [begin, end) of rank `rank`: sizes differ by at most one, earlier ranks take the remainder."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(n_items, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard(items: Sequence, rank: int, world: int) -> List:
    b, e = shard_bounds(len(items), rank, world)
    return list(items[b:e])


def round_robin(items: Sequence, rank: int, world: int) -> List:
    """Frame i goes to GPU i mod world (keeps the per-GPU mix of camera heights of a stream balanced)."""
    return list(items[rank::world])


def reduce_timing(dist, elapsed_s: float, frames: int, points: int, device=None):
    """(max elapsed over ranks, total frames, total points). `dist` is torch.distributed or None for one process."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return elapsed_s, frames, points
    import torch
    t = torch.tensor([elapsed_s], dtype=torch.float64, device=device)
    c = torch.tensor([float(frames), float(points)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(c, op=dist.ReduceOp.SUM)
    return float(t[0]), int(c[0]), int(c[1])

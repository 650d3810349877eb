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


def max_over_ranks(dist, x: float, device=None) -> float:
    """The largest x of all ranks (a timed region lasts as long as its slowest rank). `dist` is torch.distributed, or
    None for one process; `device` is where the one-element tensor lives ("cuda" for NCCL, None for gloo)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(x)
    import torch
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(dist, x: float, device=None) -> float:
    """The sum of x over all ranks (whole-job counts: frames, points, bytes)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(x)
    import torch
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())

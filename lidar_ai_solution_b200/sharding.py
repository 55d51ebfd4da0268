"""Frame sharding across GPUs: frames are independent, so ranks share nothing.

Each rank draws its own frames (disjoint seeds) and runs them on its own GPU.
The only communication is around the timed region: a barrier before it and a
max-reduction of the elapsed device time after it.
"""
from __future__ import annotations


def frame_seeds(rank: int, frames_per_rank: int, base: int = 1000):
    """Seeds of the frames rank ``rank`` processes; disjoint between ranks."""
    start = base * (rank + 1)
    if frames_per_rank > base:
        raise ValueError("at most %d frames per rank" % base)
    return list(range(start, start + frames_per_rank))


def assign_frames(voxel_counts, world: int):
    """Longest-processing-time-first assignment of a fixed set of frames to
    ``world`` ranks (used when a given list of frames, not a per-rank quota,
    has to be spread).  Returns a list of index lists, one per rank."""
    order = sorted(range(len(voxel_counts)), key=lambda i: -voxel_counts[i])
    load = [0] * world
    out = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += voxel_counts[i]
    return out


def aggregate(elapsed_ms: float, frames_done: int, dist=None, device=None):
    """(max elapsed over ranks, total frames over ranks).  ``dist`` is
    ``torch.distributed`` when a process group exists, else None."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(elapsed_ms), int(frames_done)
    import torch
    t = torch.tensor([float(elapsed_ms)], dtype=torch.float64, device=device)
    f = torch.tensor([int(frames_done)], dtype=torch.int64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(f, op=dist.ReduceOp.SUM)
    return float(t.item()), int(f.item())


def gather_floats(value: float, dist=None, device=None):
    """[value of rank 0, value of rank 1, ...] on every rank (one element without a group)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return [float(value)]
    import torch
    mine = torch.tensor([float(value)], dtype=torch.float64, device=device)
    out = [torch.zeros_like(mine) for _ in range(dist.get_world_size())]
    dist.all_gather(out, mine)
    return [float(t.item()) for t in out]

"""Scene sharding across the GPUs of one box: independent scenes, one process per GPU, no data-path
collective.  The only communication is the reduction of the timing and of the unit counts."""


def scenes_for_rank(n_scenes, rank, world):
    """Round-robin assignment: scene i runs on rank i % world."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    return list(range(rank, n_scenes, world))


def aggregate(dist, device, local_units, local_ms):
    """(total units over all ranks, max step time over ranks).  `dist` is torch.distributed (initialised)
    or None for a single process."""
    if dist is None:
        return float(local_units), float(local_ms)
    import torch
    u = torch.tensor([float(local_units)], dtype=torch.float64, device=device)
    t = torch.tensor([float(local_ms)], dtype=torch.float64, device=device)
    dist.all_reduce(u, op=dist.ReduceOp.SUM)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(u.item()), float(t.item())

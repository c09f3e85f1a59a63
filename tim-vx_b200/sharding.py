"""Batch sharding of the inference path across the GPUs of one box.

N is the slowest tim::vx dimension (shape [W,H,C,N]), so a batch shard is one
contiguous byte range of every activation tensor.  Each rank owns a full
replica of the network on its own GPU and runs its range; there is no
collective on the data path — the only communication is the optional gather of
the (tiny) outputs and, in the benchmark, the MAX-reduction of elapsed times.
The reference has the same shape of scale-out: one executor per device, whole
graphs per task (src/tim/vx/platform/native.cc:224-268).
"""


def shard_range(n_items, rank, world):
    """Items [begin, end) of rank `rank`; the remainder goes to the first ranks."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    base, rem = divmod(n_items, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def shard_bytes(array_bytes, n_items, rank, world):
    """Byte range of a batch-major buffer that belongs to `rank`."""
    per_item = array_bytes // n_items
    b, e = shard_range(n_items, rank, world)
    return b * per_item, e * per_item


def max_over_ranks(value, dist=None, device=None):
    """Largest `value` over all ranks (the slowest rank defines a step's time)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_outputs(local, n_items, dist=None):
    """All ranks' output rows concatenated in rank order (numpy uint8 [items_local, ...])."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return local
    import numpy as np
    import torch
    world = dist.get_world_size()
    width = int(np.prod(local.shape[1:])) if local.ndim > 1 else 1
    counts = [shard_range(n_items, r, world) for r in range(world)]
    biggest = max(e - b for b, e in counts)
    pad = np.zeros((biggest, width), np.uint8)
    pad[: local.shape[0]] = local.reshape(local.shape[0], width)
    bufs = [torch.empty((biggest, width), dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(bufs, torch.from_numpy(pad))
    parts = [bufs[r][: e - b].numpy() for r, (b, e) in enumerate(counts)]
    return np.concatenate(parts, axis=0).reshape((n_items,) + local.shape[1:])

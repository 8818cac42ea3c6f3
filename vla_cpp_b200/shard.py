"""Host-side sharding of independent observations over the GPUs of one box.

The denoise path has no cross-observation state (one predict = one observation in the reference,
src/model.h:204-225), so each rank gets a contiguous block of the observation list, a full weight
replica and its own KV pages; no collective runs on the data path.  torch.distributed is used only
to agree on timings (max over ranks) and, optionally, to gather the finished action chunks."""
import torch
import torch.distributed as dist


def shard_range(n_total, world, rank):
    """Contiguous block [start, start + count) of rank `rank`; the first n_total % world ranks get one extra."""
    import ctypes as C

    from .api import lib

    start, count = C.c_int64(0), C.c_int64(0)
    if lib().vlab200_shard_range(C.c_int64(n_total), int(world), int(rank), C.byref(start), C.byref(count)) != 0:
        raise ValueError("bad sharding arguments")
    return start.value, count.value


def max_over_ranks(values, device="cpu"):
    """Element-wise maximum of a list of floats over all ranks (identity without a process group)."""
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def gather_action_chunks(x_local, n_total):
    """All ranks' action chunks [count_r, chunk, A] -> [n_total, chunk, A] in observation order, on every rank.
    This is the only collective of the multi-GPU path and it runs after the loop."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return x_local
    world, rank = dist.get_world_size(), dist.get_rank()
    counts = [shard_range(n_total, world, r)[1] for r in range(world)]
    if x_local.shape[0] != counts[rank]:
        raise ValueError("local block does not match the sharding of n_total")
    width = max(counts)
    padded = x_local.new_zeros((width,) + tuple(x_local.shape[1:]))
    padded[: counts[rank]] = x_local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    return torch.cat([p[:c] for p, c in zip(parts, counts)], dim=0)

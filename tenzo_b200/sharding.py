"""Data-parallel sharding of independent decode sequences across GPUs (one process per GPU).

Sequences never interact, so there is no data-path collective: rank r decodes a contiguous slice of
the global batch with a full copy of the weights, and only timings / token ids are gathered.
"""
from __future__ import annotations


def shard_sequences(global_batch: int, world_size: int, rank: int) -> tuple[int, int]:
    """(first sequence, number of sequences) for `rank`; the first `global_batch % world_size` ranks take one extra."""
    if world_size <= 0 or not 0 <= rank < world_size or global_batch < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(global_batch, world_size)
    count = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first, count


def max_over_ranks(value: float, device=None) -> float:
    """Slowest rank's time (the number a multi-GPU measurement reports); identity without a process group."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device or ("cuda" if dist.get_backend() == "nccl" else "cpu"))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())

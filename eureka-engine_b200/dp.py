"""Stream data-parallel plumbing: independent request streams, one engine replica per GPU, no
collective on the data path.  torch.distributed is used only to agree on the timing window and to
add up what the ranks emitted (works with nccl on GPUs and with gloo on CPUs)."""
from __future__ import annotations

from typing import List, Sequence, Tuple


def shard_streams(n_streams: int, rank: int, world: int) -> List[int]:
    """Stream ids served by `rank`: round-robin, so ranks differ by at most one stream."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    return list(range(rank, n_streams, world))


def aggregate(times: Sequence[float], counts: Sequence[float], device=None) -> Tuple[List[float], List[float]]:
    """MAX over ranks of every entry of `times`, SUM over ranks of every entry of `counts`.
    Without an initialised process group the inputs come back unchanged (one rank)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(times), list(counts)
    t = torch.tensor(list(times), dtype=torch.float64, device=device)
    c = torch.tensor(list(counts), dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(c, op=dist.ReduceOp.SUM)
    return t.tolist(), c.tolist()

"""Data-parallel sharding of a subgame batch over the GPUs of one node.

Subgames are independent, so a batch is split into contiguous blocks of roots, one block
per rank, and solved with no communication.  The only exchange is at the end: the value
targets of all shards are gathered and the exploitability statistics reduced (upstream
keeps these in `RebelBatch.value_targets` and `evaluator.stats`,
p2/search/cfr_evaluator.py:1384-1495, 1652-1672).  Works with any torch.distributed
backend (NCCL over NVLink on GPUs, gloo on CPU for tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(total: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) of the contiguous block of `total` items owned by `rank`; the first
    `total % world` ranks hold one extra item."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of size {world}")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def gather_rows(local: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenates the per-rank tensors along dim 0 in rank order on every rank.  Row
    counts may differ between ranks (they are exchanged first and shards are padded to the
    largest one for the collective)."""
    if not dist.is_available() or not dist.is_initialized():
        return local
    world = dist.get_world_size(group)
    if world == 1:
        return local
    counts = torch.zeros(world, dtype=torch.int64, device=local.device)
    counts[dist.get_rank(group)] = local.shape[0]
    dist.all_reduce(counts, group=group)
    counts = counts.tolist()
    biggest = max(counts)
    if all(c == biggest for c in counts):
        out = local.new_empty((world * biggest, *local.shape[1:]))
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = local.new_zeros((biggest, *local.shape[1:]))
    padded[: local.shape[0]] = local
    out = local.new_empty((world * biggest, *local.shape[1:]))
    dist.all_gather_into_tensor(out, padded, group=group)
    return torch.cat([out[r * biggest: r * biggest + c] for r, c in enumerate(counts)], dim=0)


def reduce_exploitability(local_exploitability: torch.Tensor, group=None) -> dict:
    """mean / min / max of the per-subgame local exploitability over all ranks."""
    x = local_exploitability.detach().double()
    acc = torch.stack([x.sum(), torch.tensor(float(x.numel()), dtype=torch.float64, device=x.device)])
    if x.numel():
        lo, hi = x.min().reshape(1), x.max().reshape(1)
    else:
        lo = torch.full((1,), float("inf"), dtype=torch.float64, device=x.device)
        hi = torch.full((1,), float("-inf"), dtype=torch.float64, device=x.device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(acc, group=group)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
    count = acc[1].item()
    return {"local_exploitability": acc[0].item() / count if count else float("nan"),
            "local_exploitability_min": lo.item(), "local_exploitability_max": hi.item(), "count": int(count)}

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


def _is_distributed(group=None) -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


def gather_rows(local: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenates the per-rank tensors along dim 0 in rank order on every rank.  Row
    counts may differ between ranks (they are exchanged first and shards are padded to the
    largest one for the collective); the trailing dimensions and the dtype must agree, and a
    rank whose shard disagrees makes every rank raise ValueError instead of gathering garbage."""
    if not _is_distributed(group):
        return local
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    # one small exchange: rows, number of trailing dimensions, their sizes (up to 6), a dtype tag
    if local.dim() < 1 or local.dim() > 7:
        raise ValueError("gather_rows handles tensors of 1 to 7 dimensions")
    meta = torch.zeros(world, 9, dtype=torch.int64, device=local.device)
    mine = [local.shape[0], local.dim() - 1, *local.shape[1:]]
    meta[rank, : len(mine)] = torch.tensor(mine, dtype=torch.int64)
    meta[rank, 8] = sum(ord(ch) for ch in str(local.dtype))
    dist.all_reduce(meta, group=group)
    meta = meta.tolist()
    if any(row[1:] != meta[0][1:] for row in meta):
        raise ValueError(f"shards disagree on trailing shape or dtype: rank {rank} holds {tuple(local.shape)} "
                         f"{local.dtype}; (rows, ndim-1, dims..., dtype tag) per rank = {meta}")
    counts = [row[0] for row in meta]
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


def gather_payload(payload: dict, group=None) -> dict:
    """The training targets of one batch, gathered over the ranks: every tensor of `payload`
    (value targets [n,2,1326], beliefs [n,2652], boards, policy targets [n_pol,1326,A], ...:
    the fields of the upstream `RebelBatch`, src/p2/rl/rebel_batch.py:16-68) goes through
    `gather_rows`; other entries are passed through."""
    return {k: (gather_rows(v, group) if torch.is_tensor(v) else v) for k, v in payload.items()}


def reduce_exploitability(local_exploitability: torch.Tensor, group=None) -> dict:
    """mean / min / max of the per-subgame local exploitability over all ranks: one collective
    (an all-gather of four numbers per rank) and one device-to-host read."""
    x = local_exploitability.detach().double()
    if x.numel():
        mine = torch.stack([x.sum(), x.new_tensor(float(x.numel())), x.min(), x.max()])
    else:
        mine = x.new_tensor([0.0, 0.0, float("inf"), float("-inf")])
    if _is_distributed(group):
        allr = mine.new_empty(dist.get_world_size(group) * 4)
        dist.all_gather_into_tensor(allr, mine, group=group)
        rows = allr.view(-1, 4).tolist()
    else:
        rows = [mine.tolist()]
    total, count = sum(r[0] for r in rows), sum(r[1] for r in rows)
    return {"local_exploitability": total / count if count else float("nan"),
            "local_exploitability_min": min(r[2] for r in rows), "local_exploitability_max": max(r[3] for r in rows),
            "count": int(count)}

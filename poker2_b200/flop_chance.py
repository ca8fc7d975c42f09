"""Flop chance node on the GPU: expected leaf values over the three-card flop, the counterpart
of `ChanceNodeHelper.flop_chance_values` (p2/search/chance_node_helper.py:83-357).

The 22,100 flops fall into 1,755 suit-isomorphism classes; one canonical flop per class is
evaluated, weighted by the class size (all of them, or a sample drawn with probability
proportional to the class size), and the leaf values of a canonical flop are averaged over
its suit orbit by permuting the hand axis (all 24 suit permutations, or a random subset).
The class tables are small integer tables built on the host; the belief expansion and the
orbit average are this library's kernels; the value function (the network) is the caller's.
Random draws follow the upstream sequence of generator calls.
"""
from __future__ import annotations

from functools import lru_cache
from itertools import combinations, permutations

import numpy as np
import torch

from . import _lib

NUM_HANDS = _lib.NUM_HANDS


@lru_cache(maxsize=1)
def combo_perm_table() -> np.ndarray:
    """[24,1326] int32: the combo each combo becomes under each suit permutation
    (p2/env/card_utils.py:153-181)."""
    c1, c2 = np.triu_indices(52, k=1)
    lookup = np.full((52, 52), -1, dtype=np.int64)
    lookup[c1, c2] = np.arange(NUM_HANDS)
    out = np.empty((24, NUM_HANDS), dtype=np.int32)
    for p, perm in enumerate(np.array(tuple(permutations(range(4))), dtype=np.int64)):
        a, b = perm[c1 // 13] * 13 + c1 % 13, perm[c2 // 13] * 13 + c2 % 13
        out[p] = lookup[np.minimum(a, b), np.maximum(a, b)]
    return out


@lru_cache(maxsize=1)
def canonical_flops():
    """(cards [1755,3] int64, counts [1755] int64), ids in ascending order of the canonical code
    (chance_node_helper.py:83-180): per flop, cards sorted by rank descending, suits relabelled by
    each of the 24 suit permutations and sorted inside equal-rank groups, smallest base-52 code."""
    flops = np.array(list(combinations(range(52), 3)), dtype=np.int64)
    ranks, suits = flops % 13, flops // 13
    order = np.argsort(-ranks, axis=1, kind="stable")
    rs = np.take_along_axis(ranks, order, axis=1)
    eq01, eq12 = rs[:, 0] == rs[:, 1], rs[:, 1] == rs[:, 2]
    trips, first2, last2 = eq01 & eq12, eq01 & ~eq12, eq12 & ~eq01
    best = None
    for perm in np.array(tuple(permutations(range(4))), dtype=np.int64):
        s = np.take_along_axis(perm[suits], order, axis=1)
        s[trips] = np.sort(s[trips], axis=1)
        s[first2, :2] = np.sort(s[first2, :2], axis=1)
        s[last2, 1:] = np.sort(s[last2, 1:], axis=1)
        code = s * 13 + rs
        scalar = code[:, 0] * 2704 + code[:, 1] * 52 + code[:, 2]
        best = scalar if best is None else np.minimum(best, scalar)
    uniq, inverse = np.unique(best, return_inverse=True)
    cards = np.stack([uniq // 2704, (uniq // 52) % 52, uniq % 52], axis=1)
    return cards, np.bincount(inverse, minlength=uniq.shape[0]).astype(np.int64)


def expand_on_boards(pre_beliefs: torch.Tensor, boards: torch.Tensor) -> torch.Tensor:
    """pre_beliefs [B,2,W] fp32 (W = 1326 or padded), boards [F,L] int64 -> [B*F,2,1326]: the
    beliefs of every root re-blocked and re-normalised on every board (root-major)."""
    _lib.require_cuda(pre_beliefs, "expand_on_boards")
    assert pre_beliefs.dtype == torch.float32 and pre_beliefs.stride(2) == 1
    assert pre_beliefs.stride(0) == 2 * pre_beliefs.stride(1)
    boards = boards.to(device=pre_beliefs.device, dtype=torch.int64).contiguous()
    B, F = pre_beliefs.shape[0], boards.shape[0]
    post = torch.empty(B * F, 2, NUM_HANDS, device=pre_beliefs.device, dtype=torch.float32)
    with torch.cuda.device(pre_beliefs.device):
        _lib.call("p2b_expand_on_boards", _lib.ptr(pre_beliefs), pre_beliefs.stride(1), _lib.ptr(boards), boards.shape[1],
                  B, F, _lib.ptr(post), _lib.stream_ptr(pre_beliefs.device))
    return post


def mean_over_hand_perms(values: torch.Tensor, perms: torch.Tensor) -> torch.Tensor:
    """values [...,1326] fp32 contiguous, perms [P,1326] int32 -> mean over p of values[..., perms[p]]."""
    _lib.require_cuda(values, "mean_over_hand_perms")
    assert values.dtype == torch.float32 and values.is_contiguous() and values.shape[-1] == NUM_HANDS
    perms = perms.to(device=values.device, dtype=torch.int32).contiguous()
    out = torch.empty_like(values)
    with torch.cuda.device(values.device):
        _lib.call("p2b_mean_over_hand_perms", _lib.ptr(values), _lib.ptr(perms), perms.shape[0],
                  values.numel() // NUM_HANDS, _lib.ptr(out), _lib.stream_ptr(values.device))
    return out


def flop_chance_values(pre_beliefs: torch.Tensor, value_fn, generator: torch.Generator | None = None, *,
                       sample_size: int = 256, num_perm_samples: int = 6, chunk: int = 128) -> torch.Tensor:
    """Expected values over the flop for every root: pre_beliefs [B,2,1326(+pad)] on the device,
    value_fn(post_beliefs [S,2,1326], boards [S,5], root [S]) -> [S,2,1326].  `generator` is
    consulted as upstream does (multinomial for the flop sample, then randperm for the suit
    permutations of every evaluated chunk); it may live on the CPU."""
    device = pre_beliefs.device
    B = pre_beliefs.shape[0]
    cards_np, counts_np = canonical_flops()
    gen_device = generator.device if generator is not None else torch.device("cpu")
    canon = torch.from_numpy(cards_np).to(device)
    counts = torch.from_numpy(counts_np)
    perm_table = torch.from_numpy(combo_perm_table()).to(device)
    F = canon.shape[0]

    def eval_chunk(flops: torch.Tensor) -> torch.Tensor:
        n = flops.shape[0]
        boards5 = torch.cat([flops, torch.full((n, 2), -1, dtype=torch.long, device=device)], dim=1)
        post = expand_on_boards(pre_beliefs, boards5)
        root = torch.arange(B, device=device)[:, None].expand(-1, n).reshape(-1)
        vals = value_fn(post, boards5[None].expand(B, -1, -1).reshape(-1, 5), root).to(torch.float32).contiguous()
        if 0 < num_perm_samples < 24:
            pidx = torch.randperm(24, generator=generator, device=gen_device)[:num_perm_samples].to(device)
        else:
            pidx = torch.arange(24, device=device)
        return mean_over_hand_perms(vals, perm_table[pidx]).view(B, n, 2, NUM_HANDS)

    if 0 < sample_size < F:
        idx = torch.multinomial(counts.to(gen_device).float(), sample_size, replacement=True, generator=generator)
        return eval_chunk(canon[idx.to(device)]).mean(dim=1)
    total = torch.zeros(B, 2, NUM_HANDS, device=device)
    for a in range(0, F, chunk):
        b = min(a + chunk, F)
        weights = counts[a:b].to(device).view(1, -1, 1, 1).float()
        total += (eval_chunk(canon[a:b]) * weights).sum(dim=1)
    return total / float(counts.sum())

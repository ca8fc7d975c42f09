"""CPU oracle of the flop chance expectation.  Test infrastructure only.

Restates p2/search/chance_node_helper.py:83-357 with numpy / torch CPU ops: the canonical
flops (one representative per suit-isomorphism class of the 22,100 flops, with the class
sizes), the hole-card index permutation of every suit permutation
(p2/env/card_utils.py:153-181), and `flop_chance_values`: block and renormalise the beliefs
on every canonical flop (all of them weighted by class size, or a sample drawn with
probability proportional to class size), evaluate the value function, average the values
over the suit orbit of each flop (all 24 permutations, or a random subset) and over the flops.
"""
from __future__ import annotations

from itertools import combinations, permutations

import numpy as np
import torch

from . import cards

H = cards.NUM_HANDS


def suit_permutations() -> np.ndarray:
    return np.array(tuple(permutations(range(4))), dtype=np.int64)  # [24,4]


def combo_perm() -> np.ndarray:
    """[24,1326]: index of the combo each combo becomes under each suit permutation."""
    c1, c2 = np.triu_indices(52, k=1)
    lookup = np.full((52, 52), -1, dtype=np.int64)
    lookup[c1, c2] = np.arange(H)
    out = np.empty((24, H), dtype=np.int64)
    for p, perm in enumerate(suit_permutations()):
        a = perm[c1 // 13] * 13 + c1 % 13
        b = perm[c2 // 13] * 13 + c2 % 13
        out[p] = lookup[np.minimum(a, b), np.maximum(a, b)]
    return out


def canonical_flops():
    """(cards [F,3], counts [F]) in the order of the upstream ids: ascending canonical code."""
    flops = np.array(list(combinations(range(52), 3)), dtype=np.int64)  # [22100,3]
    ranks, suits = flops % 13, flops // 13
    order = np.argsort(-ranks, axis=1, kind="stable")
    ranks_sorted = np.take_along_axis(ranks, order, axis=1)
    eq01 = ranks_sorted[:, 0] == ranks_sorted[:, 1]
    eq12 = ranks_sorted[:, 1] == ranks_sorted[:, 2]
    best = None
    for perm in suit_permutations():
        s = np.take_along_axis(perm[suits], order, axis=1)
        all_eq, first2, last2 = eq01 & eq12, eq01 & ~eq12, eq12 & ~eq01
        s[all_eq] = np.sort(s[all_eq], axis=1)
        s[first2, :2] = np.sort(s[first2, :2], axis=1)
        s[last2, 1:] = np.sort(s[last2, 1:], axis=1)
        code = s * 13 + ranks_sorted
        scalar = code[:, 0] * 2704 + code[:, 1] * 52 + code[:, 2]
        best = scalar if best is None else np.minimum(best, scalar)
    uniq, inverse = np.unique(best, return_inverse=True)
    canon = np.stack([uniq // 2704, (uniq // 52) % 52, uniq % 52], axis=1)
    counts = np.bincount(inverse, minlength=uniq.shape[0])
    return canon, counts


def flop_chance_values(pre_beliefs: torch.Tensor, value_fn, generator: torch.Generator | None = None, *,
                       sample_size: int = 256, num_perm_samples: int = 6, chunk: int = 128) -> torch.Tensor:
    """pre_beliefs [B,2,1326]; value_fn(post_beliefs [S,2,1326], boards [S,5], root [S]) -> [S,2,1326]."""
    B = pre_beliefs.shape[0]
    canon_np, counts_np = canonical_flops()
    canon, counts = torch.from_numpy(canon_np), torch.from_numpy(counts_np)
    perm_table = torch.from_numpy(combo_perm())
    F = canon.shape[0]

    def eval_chunk(flops):
        n = flops.shape[0]
        boards5 = torch.cat([flops, torch.full((n, 2), -1, dtype=torch.long)], dim=1)
        allowed = torch.from_numpy(cards.allowed_mask(boards5.numpy()))  # [n,1326]
        allowed_b = allowed[None, :, None, :].expand(B, n, 2, H)
        post = pre_beliefs[:, None].expand(-1, n, -1, -1).clone()
        post[~allowed_b] = 0.0
        sums = post.sum(dim=-1, keepdim=True)
        uniform = allowed_b.float()
        uniform = uniform / uniform.sum(dim=-1, keepdim=True).clamp(min=1.0)
        post = torch.where(sums > 1e-12, post / sums.clamp(min=1e-12), uniform)
        root = torch.arange(B)[:, None].expand(-1, n).reshape(-1)
        vals = value_fn(post.reshape(B * n, 2, H), boards5[None].expand(B, -1, -1).reshape(-1, 5), root)
        vals = vals.float().view(B, n, 2, H)
        if 0 < num_perm_samples < 24:
            pidx = torch.randperm(24, generator=generator)[:num_perm_samples]
        else:
            pidx = torch.arange(24)
        perms = perm_table[pidx]
        g = vals.index_select(-1, perms.reshape(-1))
        return g.view(B, n, 2, perms.shape[0], H).mean(dim=-2)

    if 0 < sample_size < F:
        idx = torch.multinomial(counts.float(), sample_size, replacement=True, generator=generator)
        return eval_chunk(canon[idx]).mean(dim=1)
    total = torch.zeros(B, 2, H)
    for a in range(0, F, chunk):
        b = min(a + chunk, F)
        total += (eval_chunk(canon[a:b]) * counts[a:b].view(1, -1, 1, 1).float()).sum(dim=1)
    return total / float(counts.sum())

"""CPU oracle of the single-card chance expectation.  Test infrastructure only.

Restates p2/search/chance_node_helper.py:383-477 with torch CPU ops: enumerate the cards
not on the board (root-major, ascending card id), extend the board, zero the beliefs of
combos touching the extended board, renormalise (uniform fallback at mass <= 1e-12),
evaluate the value function, `index_add_` per root and divide by the sample count.
"""
from __future__ import annotations

import torch

from . import cards


def expand_next_card(pre_beliefs: torch.Tensor, boards: torch.Tensor):
    B = boards.shape[0]
    available = torch.ones(B, 52, dtype=torch.bool)
    for slot in range(boards.shape[1]):
        c = boards[:, slot]
        ok = c >= 0
        available[ok, c[ok]] = False
    flat = torch.nonzero(available.view(-1), as_tuple=False).squeeze(1)
    root_lookup = torch.arange(B).unsqueeze(1).expand(-1, 52).reshape(-1)[flat]
    card_values = torch.arange(52).unsqueeze(0).expand(B, -1).reshape(-1)[flat]
    S = flat.numel()
    samples = boards[root_lookup].clone()
    samples[torch.arange(S), (samples >= 0).sum(dim=1)] = card_values
    allowed = torch.from_numpy(cards.allowed_mask(samples.numpy()))
    post = pre_beliefs[root_lookup].clone()
    post.masked_fill_(~allowed.unsqueeze(1), 0.0)
    sums = post.sum(dim=-1, keepdim=True)
    uniform = allowed.unsqueeze(1).float()
    uniform = uniform / uniform.sum(dim=-1, keepdim=True).clamp(min=1.0)
    post = torch.where(sums > 1e-12, post / sums.clamp(min=1e-12), uniform)
    return post, root_lookup, samples


def single_card_chance_values(pre_beliefs, boards, value_fn):
    post, lookup, samples = expand_next_card(pre_beliefs, boards)
    values = value_fn(post, samples, lookup).float()
    B = boards.shape[0]
    total = torch.zeros(B, 2, cards.NUM_HANDS)
    counts = torch.zeros(B)
    total.index_add_(0, lookup, values)
    counts.index_add_(0, lookup, torch.ones(lookup.numel()))
    return total / counts.clamp(min=1.0).view(-1, 1, 1)

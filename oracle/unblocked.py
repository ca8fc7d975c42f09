"""CPU oracle of the unblocked-mass helper.  Test infrastructure only.

p2/env/card_utils.py:196-222: out[..., h] = sum of target over the combos that share no
card with h, computed as an fp64 product with the 1326x1326 compatibility matrix, rounded
to fp32 and clamped at zero.
"""
from __future__ import annotations

import functools

import torch

from . import cards


@functools.lru_cache(maxsize=None)
def _compat_f64() -> torch.Tensor:
    return torch.from_numpy(cards.compatible()).double()


def unblocked_mass(target: torch.Tensor) -> torch.Tensor:
    flat = target.reshape(-1, cards.NUM_HANDS)
    out = (flat.double() @ _compat_f64()).float()
    return out.view_as(target).clamp(min=0.0)

"""Card and hole-card-combo tables of the oracle (numpy).

Card id = suit*13 + rank, rank 0..12 = 2..A (p2/env/rules.py:11).  The 1326 combos are
the pairs (c1 < c2) in lexicographic order (p2/env/card_utils.py:58-68).
"""
from __future__ import annotations

import functools

import numpy as np

NUM_HANDS = 1326
NUM_CARDS = 52


@functools.lru_cache(maxsize=None)
def combos() -> np.ndarray:
    """[1326, 2] int64 card ids of every combo."""
    out = [(a, b) for a in range(NUM_CARDS) for b in range(a + 1, NUM_CARDS)]
    return np.asarray(out, dtype=np.int64)


@functools.lru_cache(maxsize=None)
def combo_lookup() -> np.ndarray:
    """[52, 52] int64, combo index of an unordered pair, -1 on the diagonal
    (p2/env/card_utils.py:71-81)."""
    table = np.full((NUM_CARDS, NUM_CARDS), -1, dtype=np.int64)
    cmb = combos()
    table[cmb[:, 0], cmb[:, 1]] = np.arange(NUM_HANDS)
    table[cmb[:, 1], cmb[:, 0]] = np.arange(NUM_HANDS)
    return table


@functools.lru_cache(maxsize=None)
def combo_onehot() -> np.ndarray:
    """[1326, 52] bool incidence of combos and cards (p2/env/card_utils.py:114-122)."""
    m = np.zeros((NUM_HANDS, NUM_CARDS), dtype=bool)
    cmb = combos()
    m[np.arange(NUM_HANDS), cmb[:, 0]] = True
    m[np.arange(NUM_HANDS), cmb[:, 1]] = True
    return m


@functools.lru_cache(maxsize=None)
def compatible() -> np.ndarray:
    """[1326, 1326] bool, True where two combos share no card
    (p2/env/card_utils.py:145-149)."""
    oh = combo_onehot().astype(np.int32)
    return (oh @ oh.T) == 0


def allowed_mask(boards: np.ndarray) -> np.ndarray:
    """[M, 1326] bool, True where the combo does not use a board card; board entries < 0
    are ignored (p2/search/cfr_evaluator.py:811-815)."""
    boards = np.asarray(boards)
    oh = combo_onehot()
    out = np.ones((boards.shape[0], NUM_HANDS), dtype=bool)
    for j in range(boards.shape[1]):
        col = boards[:, j]
        valid = col >= 0
        hit = np.zeros_like(out)
        hit[valid] = oh[:, col[valid]].T
        out &= ~hit
    return out

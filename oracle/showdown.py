"""CPU oracle of the river showdown evaluator.  Test infrastructure only.

Restates p2/search/cfr_evaluator.py:406-482 (`_init_hand_rank_data`: strength order, tie
groups) and :492-601 (`_showdown_value`: rank-CDF with per-card blocker correction) with
the same floating-point operations in the same order, so that results agree with the
upstream CPU path to the last bit on the same inputs: fp32 tensors, `torch.cumsum`
(which accumulates in fp64 on the CPU and rounds every prefix to fp32), fp32 differences.
"""
from __future__ import annotations

import numpy as np
import torch

from . import cards, rank7

H = cards.NUM_HANDS


def tie_groups(scores: np.ndarray, order: np.ndarray):
    """For every sorted position k, the half-open span [L,R) of positions holding the same
    strength (cfr_evaluator.py:428-447)."""
    m = scores.shape[0]
    L = np.empty((m, H), dtype=np.int64)
    R = np.empty((m, H), dtype=np.int64)
    for b in range(m):
        s = scores[b][order[b]]
        start = np.concatenate([[True], s[1:] != s[:-1]])
        first = np.flatnonzero(start)
        gid = np.cumsum(start) - 1
        L[b] = first[gid]
        R[b] = np.concatenate([first[1:], [H]])[gid]
    return L, R


def sorted_ev(boards, opp_beliefs, rank_mode: int = rank7.MODE_PLANES):
    """The sorted-order stage of `_showdown_value` (cfr_evaluator.py:532-596) on its own: for boards [M,5] and
    opponent beliefs [M,1326] fp32 (zero on the hands that use a board card), returns a dict with the
    inputs of that stage (`b_sorted`, `c1_sorted`, `c2_sorted`, `L`, `R`, all [M,1326], and `order`) and its
    result `ev_sorted` (win - loss as fractions of den, before the inverse permutation, the hand mask and the
    pot scaling), computed like `showdown_values` below."""
    boards = np.asarray(boards)
    x_all = torch.as_tensor(opp_beliefs, dtype=torch.float32)
    m = boards.shape[0]
    scores, order = rank7.rank_hands(boards, rank_mode)
    L_np, R_np = tie_groups(scores, order)
    srt, L, R = torch.from_numpy(order), torch.from_numpy(L_np), torch.from_numpy(R_np)
    cmb = torch.from_numpy(cards.combos())
    onehot = torch.from_numpy(cards.combo_onehot())
    c_sorted = cmb[srt]
    c1, c2 = c_sorted[..., 0], c_sorted[..., 1]
    x = x_all.gather(1, srt)
    ev = torch.empty(m, H, dtype=torch.float32)
    for b in range(m):
        card_ok = torch.ones(52, dtype=torch.bool)
        card_ok[torch.from_numpy(boards[b].astype(np.int64))] = False
        inc = onehot[srt[b]] & card_ok[None, :]
        xb = x[b]
        P = torch.cat([torch.zeros(1), torch.cumsum(xb, dim=0)])
        PC = torch.cat([torch.zeros(1, 52), torch.cumsum(inc.float() * xb[:, None], dim=0)], dim=0)
        at = lambda pos, card: PC[pos, card]  # noqa: E731
        PL, PR = P[L[b]], P[R[b]]
        a0, b0, a1, b1 = at(L[b], c1[b]), at(L[b], c2[b]), at(R[b], c1[b]), at(R[b], c2[b])
        win = PL - a0 - b0
        tie = (PR - PL) - (a1 - a0) - (b1 - b0) + xb
        tot = PC[-1]
        den = (1.0 - tot[c1[b]] - tot[c2[b]] + xb).clamp(min=1e-8)
        ok = den > 1e-8
        wp = torch.where(ok, win / den, torch.zeros(()))
        tp = torch.where(ok, tie / den, torch.zeros(()))
        lp = torch.where(ok, 1.0 - wp - tp, torch.zeros(()))
        ev[b] = wp - lp
    return dict(b_sorted=x, c1_sorted=c1, c2_sorted=c2, L=L, R=R, order=srt, ev_sorted=ev)


def showdown_values(boards, beliefs, potential, scale, rank_mode: int = rank7.MODE_PLANES, chunk: int = 16):
    """boards [M,5] ints, beliefs [M,2,1326] fp32, potential [M,2] int64, scale [M] fp32
    -> values [M,2,1326] fp32 (value of player p's hands against beliefs[:,1-p])."""
    boards = np.asarray(boards)
    beliefs = torch.as_tensor(beliefs, dtype=torch.float32)
    potential = torch.as_tensor(potential, dtype=torch.int64)
    scale = torch.as_tensor(scale, dtype=torch.float32)
    m = boards.shape[0]
    out = torch.empty(m, 2, H, dtype=torch.float32)
    scores, order = rank7.rank_hands(boards, rank_mode)
    L_np, R_np = tie_groups(scores, order)
    allowed = torch.from_numpy(cards.allowed_mask(boards))
    cmb = torch.from_numpy(cards.combos())
    onehot = torch.from_numpy(cards.combo_onehot())
    for lo in range(0, m, chunk):
        hi = min(m, lo + chunk)
        n = hi - lo
        srt = torch.from_numpy(order[lo:hi])
        L = torch.from_numpy(L_np[lo:hi])
        R = torch.from_numpy(R_np[lo:hi])
        inv = torch.argsort(srt, dim=1)
        card_ok = torch.ones(n, 52, dtype=torch.bool)
        card_ok.scatter_(1, torch.from_numpy(boards[lo:hi].astype(np.int64)), False)
        c_sorted = cmb[srt]  # [n,1326,2]
        inc = onehot[srt] & card_ok[:, None, :]  # [n,1326,52] incidence in strength order
        for hero in range(2):
            x = beliefs[lo:hi, 1 - hero].gather(1, srt)
            zero1 = torch.zeros(n, 1)
            P = torch.cat([zero1, torch.cumsum(x, dim=1)], dim=1)
            PC = torch.cat([torch.zeros(n, 1, 52), torch.cumsum(inc.float() * x[..., None], dim=1)], dim=1)
            c1 = c_sorted[..., 0]
            c2 = c_sorted[..., 1]

            def at(pos, card):  # PC[b, pos[b,k], card[b,k]]
                return PC.gather(1, pos[..., None].expand(-1, -1, 52)).gather(2, card[..., None]).squeeze(-1)

            PL = P.gather(1, L)
            PR = P.gather(1, R)
            a0, b0 = at(L, c1), at(L, c2)
            a1, b1 = at(R, c1), at(R, c2)
            win = PL - a0 - b0
            tie = (PR - PL) - (a1 - a0) - (b1 - b0) + x
            tot = PC[:, -1, :]
            den = (1.0 - tot.gather(1, c1) - tot.gather(1, c2) + x).clamp(min=1e-8)
            ok = den > 1e-8
            wp = torch.where(ok, win / den, torch.zeros(()))
            tp = torch.where(ok, tie / den, torch.zeros(()))
            lp = torch.where(ok, 1.0 - wp - tp, torch.zeros(()))
            ev = (wp - lp).gather(1, inv) * allowed[lo:hi].float()
            out[lo:hi, hero] = ev * potential[lo:hi, hero][:, None] / scale[lo:hi, None]
    return out

"""Evaluator statistics, computed on the device with one device-to-host read per batch.

Same keys and definitions as the upstream evaluator records after a solve
(p2/search/cfr_evaluator.py: `_record_cfr_entropy` :1607-1616, `_record_cumulative_regret`
:1634-1672, `_record_action_mix` :1674-1690); the trainer merges them into its metrics
(p2/rl/cfr_trainer.py:422).  `cfr_delta.*` (the policy change at five iterations, :1574-1605) needs
the policy before and after single iterations and is not recorded here (the upstream graphed fused
evaluator skips it as well, p2/search/fused_sparse_cfr_evaluator.py:522-527).
"""
from __future__ import annotations

import numpy as np
import torch

NUM_HANDS = 1326
STREETS = ("preflop", "flop", "turn", "river", "showdown")


def evaluator_stats(res, trees, boards: np.ndarray) -> dict:
    """res: a `solver.SolveResult` with exploitability; trees: the host trees of the batch; boards
    [N,5] root boards (-1 = not dealt).  Returns the upstream statistics dictionary entries."""
    dev = res.policy_avg.device
    N, top, A = trees.num_roots, trees.depth_offsets[-2], trees.num_actions
    pol = res.level_major(res.policy_avg)
    parent = torch.from_numpy(trees.parent_index[N:]).to(dev)
    action = torch.from_numpy(trees.action_from_parent[N:]).to(dev)
    by_src = torch.zeros((top, A, NUM_HANDS), dtype=torch.float32, device=dev)
    by_src[parent, action] = pol[N:]
    non_leaf = torch.from_numpy(~trees.leaf_mask[:top]).to(dev)
    out = []
    # entropy of the average policy at the roots
    probs = by_src[:N][non_leaf[:N]]
    ent = torch.where(probs > 1e-5, -(probs * probs.clamp(min=1e-30).log()), torch.zeros((), device=dev))
    out.append(ent.sum(dim=1).mean() if probs.numel() else torch.zeros((), device=dev))
    # regret statistics
    reg = res.level_major(res.regrets).clamp(min=0)
    out.append(reg.mean())
    if res.weight_sums is not None:
        w = res.level_major(res.weight_sums)
        root_child = parent < N
        q = torch.zeros((N, A, NUM_HANDS), dtype=torch.float32, device=dev)
        q[parent[root_child], action[root_child]] = reg[N:][root_child] / w[N:][root_child]
        out.append(q.max(dim=1).values.sum(dim=1).sum() / float(N))
    else:
        out.append(torch.full((), float("nan"), device=dev))
    # local exploitability
    ex = res.exploitability
    out += [ex.mean(), ex.max(), ex.min()]
    street = torch.from_numpy(trees.state.street[:N]).to(dev)
    for i in range(len(STREETS)):
        sel = street == i
        out.append(torch.where(sel, ex, torch.zeros_like(ex)).sum() / sel.sum().clamp(min=1))
        out.append(sel.any().float())
    # action mix over the decision nodes: mean over the allowed hands of the average policy
    n_board = torch.from_numpy((np.asarray(boards) >= 0).sum(axis=1)).to(dev)
    allowed = ((52 - n_board) * (51 - n_board) // 2).to(torch.float32)[torch.from_numpy(trees.root_of[:top]).to(dev)]
    mix = by_src[non_leaf].sum(dim=2) / allowed[non_leaf][:, None]
    bet = mix[:, 2:-1].mean(dim=1).mean() if A > 3 else torch.full((), float("nan"), device=dev)
    out += [mix[:, 0].mean(), mix[:, 1].mean(), bet, mix[:, -1].mean()]
    v = torch.stack([x.reshape(()).to(torch.float32) for x in out]).cpu().tolist()  # the one read
    stats = {"cfr_entropy": v[0], "mean_positive_regret": v[1], "mean_regret_bound": v[2],
             "local_exploitability": v[3], "local_exploitability_max": v[4], "local_exploitability_min": v[5]}
    stats["local_exploitability_street"] = {STREETS[i]: v[6 + 2 * i] for i in range(len(STREETS)) if v[7 + 2 * i] > 0}
    base = 6 + 2 * len(STREETS)
    stats["action_mix"] = {"fold": v[base], "call": v[base + 1], "bet": v[base + 2], "allin": v[base + 3]}
    return stats

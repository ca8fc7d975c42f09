"""Evaluator statistics, computed on the device with one device-to-host read per batch.

Same keys and definitions as the upstream evaluator records after a solve
(p2/search/cfr_evaluator.py: `_record_cfr_entropy` :1607-1616, `_record_cumulative_regret`
:1634-1672, `_record_action_mix` :1674-1690); the trainer merges them into its metrics
(p2/rl/cfr_trainer.py:422).  `cfr_delta.*` (the policy change at five iterations, `_record_stats`
:1573-1605) needs the policy before and after single iterations: `PolicyDelta` computes it from the
cumulative regrets on either side of an iteration, for a solve that runs pass by pass (the upstream
graphed fused evaluator skips these keys, p2/search/fused_sparse_cfr_evaluator.py:522-527; here they
are recorded on request).
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


PERCENTILES = (0, 25, 50, 75, 100)


def delta_checkpoints(warm_start_iterations: int, iterations: int) -> dict:
    """Iteration -> percentile of the `cfr_delta.<percentile>` key recorded at it: the five points
    linspace(warm start, T - 1, 5), rounded as upstream rounds them (cfr_evaluator.py:1577-1589);
    where points coincide the first one names the key."""
    points = torch.linspace(int(warm_start_iterations), int(iterations) - 1, 5).round().int().tolist()
    out: dict = {}
    for q, t in zip(PERCENTILES, points):
        if int(warm_start_iterations) <= t < int(iterations):
            out.setdefault(int(t), q)
    return out


class PolicyDelta:
    """The quantity behind `cfr_delta.*` (cfr_evaluator.py:1590-1605) for one batch of trees: the absolute
    change of the current policy summed over actions and hands, counted where some player reaches the
    acting node with the hand under the new policy, divided by that node's number of such hands and
    averaged over the nodes that have any (every node above the deepest level of the batch).

    The current policy of an iteration is regret matching on the cumulative regrets
    (`update_policy`, :1168-1185), so the caller hands in the regret rows before and after the update
    of that iteration; sums run in another order than the upstream tensor reductions, which moves the
    result in the last bits only."""

    def __init__(self, trees, boards, layout, device):
        from .solver import layout_tensor

        dev = torch.device(device)
        as_t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev, torch.int64)  # noqa: E731
        self.N, self.M, self.top, self.A = trees.num_roots, trees.total_nodes, trees.depth_offsets[-2], trees.num_actions
        self.offsets = [int(x) for x in trees.depth_offsets]
        self.parent, self.action = as_t(trees.parent_index), as_t(trees.action_from_parent)
        self.prev_actor = as_t(trees.prev_actor)
        self.rows_of = layout_tensor(layout, "from_level_major", dev)
        cc = torch.from_numpy(trees.child_count[trees.parent_index.clip(min=0)]).clamp(min=1)
        self.uniform = (1.0 / cc.to(torch.float32)).to(dev)  # [M] one over the siblings of a node
        c1, c2 = np.triu_indices(52, k=1)
        hit = torch.zeros(self.N, 53, dtype=torch.bool, device=dev)
        cards = torch.from_numpy(np.asarray(boards)).to(dev, torch.int64)
        hit.scatter_(1, torch.where(cards >= 0, cards, torch.full_like(cards, 52)), True)
        allowed_root = ~(hit[:, as_t(c1)] | hit[:, as_t(c2)])
        self.allowed = allowed_root[as_t(trees.root_of)]  # [M,1326]
        self.device = dev

    def start_policy(self, start_policy: torch.Tensor | None) -> torch.Tensor:
        """The policy the first iteration moves away from: the given start policy [M,1326] (upstream node
        order), else uniform over the children of every node."""
        if start_policy is not None:
            return start_policy.to(self.device, torch.float32)
        return self.uniform[:, None].expand(-1, NUM_HANDS)

    def policy_of(self, regret_rows: torch.Tensor) -> torch.Tensor:
        """Regret matching on the solver's regret rows [rows,1344]; the result [M,1326] is in the upstream
        node order.  Sibling sums run in action order."""
        N, parent, action = self.N, self.parent[self.N:], self.action[self.N:]
        pos = regret_rows.index_select(0, self.rows_of)[..., :NUM_HANDS].clamp(min=0.0)
        sums = torch.zeros((self.top, NUM_HANDS), dtype=torch.float32, device=self.device)
        for a in range(self.A):
            sel = action == a
            sums[parent[sel]] += pos[N:][sel]
        denom = sums[parent]
        pol = torch.zeros_like(pos)
        pol[N:] = torch.where(denom > 1e-8, pos[N:] / denom.clamp(min=1e-8), self.uniform[N:, None])
        return pol

    def __call__(self, before: torch.Tensor, after: torch.Tensor) -> torch.Tensor:
        """before, after: policies [M,1326] in the upstream node order.  Returns a 0-dim device tensor."""
        N, offs = self.N, self.offsets
        reach = torch.ones((self.M, 2, NUM_HANDS), dtype=torch.float32, device=self.device)
        for d in range(len(offs) - 2):  # `_calculate_reach_weights`, cfr_evaluator.py:332-361
            b, c = offs[d + 1], offs[d + 2]
            level = reach[self.parent[b:c]].clone()
            rows = torch.arange(c - b, device=self.device)
            level[rows, self.prev_actor[b:c]] *= after[b:c]
            reach[b:c] = level
        reach.masked_fill_(~self.allowed[:, None, :], 0.0)
        reachable = (reach > 0).any(dim=1)[: self.top]
        parent = self.parent[N:]
        change = ((after[N:] - before[N:]).abs() * reachable[parent]).sum(dim=1)
        total = torch.zeros(self.top, dtype=torch.float32, device=self.device)
        for a in range(self.A):
            sel = self.action[N:] == a
            total[parent[sel]] += change[sel]
        count = reachable.sum(dim=1)
        nodes = count > 0
        delta = torch.where(nodes, total / count.clamp(min=1), torch.zeros((), device=self.device))
        return delta.sum() / nodes.sum()

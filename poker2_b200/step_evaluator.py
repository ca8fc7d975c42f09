"""The upstream evaluator's step methods, one by one, on the step-level kernels.

`StepCFREvaluator` keeps the solver state in the upstream layout (level-major over the batch, 1326
columns, the tensor names of p2/search/cfr_evaluator.py:107-170) and offers the methods the upstream
tests and tools call directly: `initialize_policy_and_beliefs`, `set_leaf_values`,
`compute_expected_values`, `compute_instantaneous_regrets`, `update_policy`, `update_average_policy`,
`cfr_iteration`, `update_average_values_final`, `evaluate_cfr`.  Each is composed from the kernels of
`poker2_b200.fused_cfr` and `poker2_b200.showdown` the way the upstream fused evaluator composes its
Triton kernels (p2/search/fused_sparse_cfr_evaluator.py:144-527), so the state can be inspected
between any two steps.  It is the slow, transparent form: a whole solve belongs in
`solver.SubgameSolver` (three launches), which ends in the same state.

Covered: uniform start, `cfr_type` standard / discounted / discounted_plus with optional CFR+ clamp,
leaves valued by showdown, fold constants and an optional `leaf_fn`; value targets from the final
average policy.  Warm starts, cfr_avg, linear CFR and running value targets are solver features
(`solver.SteppedSolver`) and are not repeated here.
"""
from __future__ import annotations

import numpy as np
import torch

from . import fused_cfr as F
from . import showdown

NUM_HANDS = 1326


class StepCFREvaluator:
    num_players = 2

    def __init__(self, trees, boards, root_beliefs: torch.Tensor, device, *, iterations: int,
                 cfr_type: str = "discounted", alpha: float = 1.5, beta: float = 0.0, gamma: float = 2.0,
                 dcfr_delay: int = 0, cfr_plus: bool = False, leaf_fn=None):
        """trees: `tree.PublicTrees`; boards [N,5] (-1 = not dealt); root_beliefs [N,2,1326];
        leaf_fn(beliefs [L,2,1326], nodes [L]) -> [L,2,1326] values of the leaves that do not end the hand."""
        if cfr_type not in ("standard", "discounted", "discounted_plus"):
            raise ValueError(f"cfr_type {cfr_type!r} is not offered step by step")
        dev = torch.device(device)
        if dev.type != "cuda":
            raise ValueError("StepCFREvaluator requires a CUDA device.")
        self.device, self.cfr_iterations = dev, int(iterations)
        self.cfr_type, self.dcfr_alpha, self.dcfr_beta, self.dcfr_gamma = cfr_type, alpha, beta, gamma
        self.dcfr_delay, self.cfr_plus, self.leaf_fn = int(dcfr_delay), bool(cfr_plus), leaf_fn
        t = trees
        as_t = lambda a, dt=torch.int64: torch.from_numpy(np.ascontiguousarray(a)).to(dev, dt)  # noqa: E731
        self.depth_offsets = [int(x) for x in t.depth_offsets]
        self.root_nodes = N = t.num_roots
        self.total_nodes = M = t.total_nodes
        self.top, self.num_actions, self.tree_depth = self.depth_offsets[-2], t.num_actions, t.tree_depth
        self.parent_index, self.action_from_parent = as_t(t.parent_index), as_t(t.action_from_parent)
        self.prev_actor, self.to_act = as_t(t.prev_actor), as_t(t.state.to_act)
        self.child_count, self.child_offsets = as_t(t.child_count), as_t(t.child_offsets)
        self.leaf_mask, self.done = as_t(t.leaf_mask, torch.bool), as_t(t.state.done, torch.bool)
        self.root_of = as_t(t.root_of)
        self.showdown_indices = torch.nonzero(as_t(t.state.street) == 4).squeeze(1)
        self.model_indices = torch.nonzero(self.leaf_mask & ~self.done).squeeze(1)
        if self.model_indices.numel() and leaf_fn is None:
            raise ValueError("the trees have leaves that do not end the hand: a leaf_fn is required")
        self._sd_potential = as_t(t.showdown_potential)[self.showdown_indices].contiguous()
        self._sd_scale = as_t(t.state.scale, torch.float32)[self.showdown_indices].contiguous()
        self._sd_table = self.root_of[self.showdown_indices].to(torch.int32).contiguous()
        boards_t = torch.from_numpy(np.asarray(boards, dtype=np.int64)).to(dev)
        self._tables = showdown.BoardTables(boards_t) if self.showdown_indices.numel() else None

        c1, c2 = np.triu_indices(52, k=1)
        hit = torch.zeros(N, 53, dtype=torch.bool, device=dev)
        hit.scatter_(1, torch.where(boards_t >= 0, boards_t, torch.full_like(boards_t, 52)), True)
        allowed_root = ~(hit[:, as_t(c1)] | hit[:, as_t(c2)])
        prob_root = allowed_root.to(torch.float32)
        prob_root = prob_root / prob_root.sum(-1, keepdim=True).clamp(min=1.0)
        self.allowed_hands = allowed_root[self.root_of].contiguous()
        self.allowed_hands_prob = prob_root[self.root_of].contiguous()

        z = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)  # noqa: E731
        self.policy_probs, self.policy_probs_avg = z(M, NUM_HANDS), z(M, NUM_HANDS)
        self.cumulative_regrets, self.regret_weight_sums = z(M, NUM_HANDS), z(M, NUM_HANDS)
        self.uniform_policy = z(M, NUM_HANDS)
        siblings = self.child_count[self.parent_index[N:]].clamp(min=1).to(torch.float32)
        self.uniform_policy[N:] = (1.0 / siblings)[:, None]
        self.beliefs = z(M, 2, NUM_HANDS)
        self.beliefs[:N] = root_beliefs.to(dev, torch.float32)[..., :NUM_HANDS]
        self.beliefs_avg = self.beliefs.clone()
        self.self_reach, self.self_reach_avg = z(M, 2, NUM_HANDS), z(M, 2, NUM_HANDS)
        self.latest_values = z(M, 2, NUM_HANDS)
        fold = (self.action_from_parent == 0) & self.done
        fv = as_t(t.fold_value, torch.float32)
        self.latest_values[fold, 0] = fv[fold][:, None]
        self.latest_values[fold, 1] = -fv[fold][:, None]
        self.values_avg = self.latest_values.clone()
        # iteration scalars on the device, so that one captured iteration can be replayed for another t
        # (fused_sparse_cfr_evaluator.py:100-107, 535-550)
        self._t_scalars = F.TScalars(dev)
        self._skip_t_scalars_update = False

    # ---- reach and beliefs (cfr_evaluator.py:248-273, 332-380) ------------------------------
    def _calculate_reach_weights(self, target: torch.Tensor, policy: torch.Tensor) -> None:
        offs = self.depth_offsets
        target.zero_()
        target[: self.root_nodes] = self.allowed_hands[: self.root_nodes, None, :].to(torch.float32)
        for d in range(self.tree_depth):
            F.fused_reach_weights_depth_(target, policy, self.allowed_hands, self.parent_index, self.prev_actor,
                                         offs[d + 1], offs[d + 2])

    def _propagate_all_beliefs(self, target: torch.Tensor, reach: torch.Tensor) -> None:
        """Every row = its root's row x reach, blocked and normalised; the root rows themselves are
        normalised once more per call, like every other row upstream."""
        N = self.root_nodes
        F.fused_deep_beliefs_(target, target, reach, self.allowed_hands_prob, self.root_of, num_roots=N)
        roots = target[:N]
        roots.mul_(reach[:N])
        F.fused_block_and_normalize_beliefs_(roots, self.allowed_hands[:N], self.allowed_hands_prob[:N])

    # ---- start of evaluate_cfr (cfr_evaluator.py:832-886, 1503-1513) ------------------------
    def initialize_policy_and_beliefs(self) -> None:
        offs, N = self.depth_offsets, self.root_nodes
        self.policy_probs.copy_(self.uniform_policy)
        for d in range(self.tree_depth):
            b, c = offs[d + 1], offs[d + 2]
            level = self.beliefs[self.parent_index[b:c]].clone()
            rows = torch.arange(c - b, device=self.device)
            level[rows, self.prev_actor[b:c]] *= self.policy_probs[b:c]
            self.beliefs[b:c] = level
            # upstream blocks and normalises the whole tensor after every level
            F.fused_block_and_normalize_beliefs_(self.beliefs, self.allowed_hands, self.allowed_hands_prob)
        if self.tree_depth == 0:
            F.fused_block_and_normalize_beliefs_(self.beliefs, self.allowed_hands, self.allowed_hands_prob)
        self._calculate_reach_weights(self.self_reach, self.policy_probs)
        self.policy_probs_avg.copy_(self.policy_probs)
        self.self_reach_avg.copy_(self.self_reach)
        self.beliefs_avg.copy_(self.beliefs)

    # ---- leaves and backup (cfr_evaluator.py:1025-1115) -------------------------------------
    def set_leaf_values(self, t: int = 0, beliefs: torch.Tensor | None = None) -> None:
        beliefs = self.beliefs if beliefs is None else beliefs
        if self.model_indices.numel():
            vals = self.leaf_fn(beliefs[self.model_indices], self.model_indices)
            self.latest_values[self.model_indices] = vals[..., :NUM_HANDS].to(torch.float32)
        if self.showdown_indices.numel():
            vals = showdown.showdown_values(self._tables, beliefs[self.showdown_indices].contiguous(), self._sd_potential,
                                            self._sd_scale, table_of_row=self._sd_table)
            self.latest_values[self.showdown_indices] = vals

    def compute_expected_values(self, policy=None, beliefs=None, leaf_values=None, values=None) -> None:
        policy = self.policy_probs if policy is None else policy
        beliefs = self.beliefs if beliefs is None else beliefs
        leaf_values = self.latest_values if leaf_values is None else leaf_values
        values = leaf_values if values is None else values
        if leaf_values is values:
            values.masked_fill_((~self.leaf_mask)[:, None, None], 0.0)
        else:
            torch.where(self.leaf_mask[:, None, None], leaf_values, torch.zeros((), device=self.device), out=values)
        N, top, offs = self.root_nodes, self.top, self.depth_offsets
        idx = self.to_act[:top, None, None].expand(-1, -1, NUM_HANDS)
        actor_beliefs = beliefs[:top].gather(1, idx).squeeze(1).contiguous()
        marginal = (actor_beliefs.index_select(0, self.parent_index[N:]) * policy[N:]).contiguous()
        opp = torch.zeros_like(policy)
        opp[N:] = F.unblocked_mass_ratio_indirect_triton(marginal, actor_beliefs, self.parent_index[N:].contiguous())
        for d in range(self.tree_depth - 1, -1, -1):
            a, b = offs[d], offs[d + 1]
            F.fused_weighted_parent_sum(values, self.prev_actor, policy, opp, self.child_offsets[a:b].contiguous(),
                                        self.child_count[a:b].contiguous(), parent_base=a, max_children=self.num_actions)

    # ---- one iteration (cfr_evaluator.py:1117-1258, 1331-1381) ------------------------------
    def compute_instantaneous_regrets(self, values: torch.Tensor | None = None) -> torch.Tensor:
        values = self.latest_values if values is None else values
        N, top = self.root_nodes, self.top
        src_weights = F.unblocked_mass_opp_at_parents_triton(self.beliefs, self.to_act, top)
        rows = torch.arange(top, device=self.device)
        actor_values = values[:top][rows, self.to_act[:top], :].contiguous()
        regrets = torch.zeros_like(self.policy_probs)
        F.fused_regret_tail_(regrets, values, actor_values, src_weights.contiguous(), self.parent_index, self.prev_actor,
                             bottom=N)
        return regrets

    def _get_mixing_weights(self, t: int):
        if self.cfr_type == "standard":
            return float(t), 1.0
        if self.cfr_type == "discounted":
            return float(t ** self.dcfr_gamma), float((t + 1) ** self.dcfr_gamma)
        return (float(t - self.dcfr_delay), 2.0) if t > self.dcfr_delay else (0.0, 1.0)

    def update_average_policy(self, t: int) -> None:
        if (self.cfr_type in ("discounted", "discounted_plus") and t <= self.dcfr_delay) or t == 0:
            self.policy_probs_avg.copy_(self.policy_probs)
            return
        N, top = self.root_nodes, self.top
        avg, ts = self.policy_probs_avg, self._t_scalars
        F.fused_average_policy_mix_with_tensors_(avg, self.policy_probs, self.self_reach, self.self_reach_avg, self.to_act,
                                                 self.parent_index, ts.mix_old, ts.mix_new, ts.mix_total, bottom=N)
        psum = F.fused_parent_sum(avg, self.child_offsets[:top].contiguous(), self.child_count[:top].contiguous(),
                                  max_children=self.num_actions)
        child = avg[N:].contiguous()
        F.fused_divide_by_parent_sum_(child, child, psum, self.parent_index[N:].contiguous(), avg[N:], eps=1e-5)
        avg[:N] = 0.0

    def update_policy(self, t: int) -> None:
        N, top = self.root_nodes, self.top
        pos = self.cumulative_regrets.clamp(min=0.0).contiguous()
        parent_sum = F.fused_parent_sum(pos, self.child_offsets[:top].contiguous(), self.child_count[:top].contiguous(),
                                        max_children=self.num_actions)
        F.fused_divide_by_parent_sum_(pos[N:].contiguous(), self.uniform_policy[N:].contiguous(), parent_sum,
                                      self.parent_index[N:].contiguous(), self.policy_probs[N:])
        self._calculate_reach_weights(self.self_reach, self.policy_probs)
        self._propagate_all_beliefs(self.beliefs, self.self_reach)
        self.update_average_policy(t)
        self._calculate_reach_weights(self.self_reach_avg, self.policy_probs_avg)
        self._propagate_all_beliefs(self.beliefs_avg, self.self_reach_avg)

    def prepare_replay(self, t: int) -> None:
        """Fills the device scalars of iteration t (discount factors, mixing weights); `cfr_iteration` does it
        itself unless `_skip_t_scalars_update` is set, which a graph capture sets so that the fills stay outside
        the captured region (fused_sparse_cfr_evaluator.py:535-550)."""
        old, new = self._get_mixing_weights(t)
        discounted = self.cfr_type in ("discounted", "discounted_plus")
        self._t_scalars.update(int(t), self.dcfr_alpha if discounted else 0.0, self.dcfr_beta if discounted else 0.0,
                               old, new)

    def cfr_iteration(self, t: int) -> None:
        if not self._skip_t_scalars_update:
            self.prepare_replay(t)
        regrets = self.compute_instantaneous_regrets(self.latest_values)
        ts = self._t_scalars
        F.fused_dcfr_update_with_tensors_(self.cumulative_regrets, self.regret_weight_sums, regrets, ts.t_alpha_num,
                                          ts.t_beta_num, ts.t_alpha_den, ts.t_beta_den,
                                          self.cfr_type in ("discounted", "discounted_plus"), self.cfr_plus)
        self.update_policy(t)
        self.set_leaf_values(t)
        self.compute_expected_values()

    def update_average_values_final(self) -> None:
        self.set_leaf_values(0, beliefs=self.beliefs_avg)
        self.compute_expected_values(self.policy_probs_avg, self.beliefs_avg, self.latest_values, self.values_avg)

    def evaluate_cfr(self) -> None:
        """The loop of cfr_evaluator.py:1497-1520 without the leaf sampling at its end."""
        self.initialize_policy_and_beliefs()
        self.set_leaf_values(0)
        self.compute_expected_values()
        self.values_avg.copy_(self.latest_values)
        for t in range(self.cfr_iterations):
            self.cfr_iteration(t)
        self.update_average_values_final()

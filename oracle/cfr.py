"""CPU oracle of the subgame CFR loop on a ragged public tree.  Test infrastructure only.

Restates, with torch CPU tensors and the same fp32 operations in the same order, the
upstream sparse evaluator (leaves: fold, showdown, or valued by a caller-supplied
`leaf_fn`, the stand-in for the value network of `set_leaf_values` :1025-1047):
p2/search/cfr_evaluator.py (`initialize_policy_and_beliefs` :830-886, `cfr_iteration`
:1331-1381, `compute_instantaneous_regrets` :1117-1165, `update_policy` :1168-1193,
`update_average_policy` :1195-1258, `compute_expected_values` :1049-1115,
`update_average_values_final` :1276-1292, `_best_response_values` /
`_compute_exploitability` :603-764) with the tree primitives of
p2/search/sparse_cfr_evaluator.py (:428-538).

The tree comes in the upstream node order: level-major over the whole batch, children of a
parent contiguous in action order.  Required keys of `tree` (numpy arrays):
  depth_offsets [D+2] int, parent_index [M], action_from_parent [M], to_act [M],
  child_count [M], leaf_mask [M] bool, done [M] bool, street [M] (4 = showdown reached),
  fold_value [M] fp32 (value for player 0 at fold leaves, 0 elsewhere),
  showdown_potential [M,2] int64, scale [M] fp32, boards [N,5], num_actions int.
The initial policy is uniform over the legal children, which is what the upstream code
obtains from a model that returns zero logits (:306-330).
"""
from __future__ import annotations

import numpy as np
import torch

from . import cards, showdown, unblocked

H = cards.NUM_HANDS


class SubgameOracle:
    def __init__(self, tree: dict, root_beliefs: torch.Tensor, *, iterations: int,
                 alpha: float = 1.5, beta: float = 0.0, gamma: float = 2.0,
                 dcfr_delay: int = 0, cfr_type: str = "discounted", cfr_plus: bool = False, leaf_fn=None,
                 start_policy: torch.Tensor | None = None, warm_start_iterations: int = 0,
                 warm_start_multiplier: float = 1.0, alpha_final: float | None = None,
                 beta_final: float | None = None, gamma_final: float | None = None,
                 enforce_zero_sum: bool = False, cfr_avg: bool = False, final_policy_values: bool = True,
                 warm_start_type: str = "model"):
        t = {k: (torch.from_numpy(np.ascontiguousarray(v)) if isinstance(v, np.ndarray) else v)
             for k, v in tree.items()}
        self.offs = [int(x) for x in tree["depth_offsets"]]
        self.N = self.offs[1]
        self.M = self.offs[-1]
        self.depth = len(self.offs) - 2
        self.top = self.offs[-2]
        self.A = int(tree["num_actions"])
        self.parent = t["parent_index"].long()
        self.action = t["action_from_parent"].long()
        self.to_act = t["to_act"].long()
        self.child_count = t["child_count"].long()
        self.leaf = t["leaf_mask"].bool()
        self.done = t["done"].bool()
        self.fold_value = t["fold_value"].float()
        self.scale = t["scale"].float()
        self.iterations = iterations
        self.alpha, self.beta, self.gamma = alpha, beta, gamma
        # exponent schedules (`apply_schedules`, cfr_evaluator.py:1294-1329) and the zero-sum shift of
        # the final values (`_maybe_enforce_zero_sum` :957-980, applied at :1289-1292)
        self.alpha0, self.beta0, self.gamma0 = alpha, beta, gamma
        self.alpha_final, self.beta_final, self.gamma_final = alpha_final, beta_final, gamma_final
        self.enforce_zero_sum = enforce_zero_sum
        # `cfr_avg` upstream (cfr_evaluator.py:997-1018, :1029, :1133): leaf values and regret weights come
        # from the beliefs under the AVERAGE policy, and from the second iteration on the model's leaf
        # values are taken as a running average and de-averaged
        self.cfr_avg = cfr_avg
        self.last_model_values = None
        # False: `value_targets_from_final_policy = False` upstream -- values_avg is a running mix of the
        # per-iteration values (`update_average_values`, :1260-1274) and no final pass recomputes it
        self.final_policy_values = final_policy_values
        self.dcfr_delay = dcfr_delay
        self.cfr_type = cfr_type
        self.cfr_plus = cfr_plus
        # leaves that are not terminal are valued by leaf_fn(beliefs[idx] [L,2,1326], idx) -> [L,2,1326]
        self.leaf_fn = leaf_fn
        # start policy [M,1326] (the policy head's softmax upstream, :306-330; None = uniform) and the
        # warm start of type `model` (:887-926): regrets seeded so that regret matching replays it
        self.start_policy = start_policy
        self.warm_start_iterations = warm_start_iterations
        self.warm_start_multiplier = warm_start_multiplier
        self.warm_start_type = warm_start_type  # "model" (:913-926) or "model_br" (:927-955)
        self.model_idx = torch.where(self.leaf & ~self.done)[0]
        N, M = self.N, self.M

        self.prev_actor = torch.full((M,), -1, dtype=torch.long)
        self.prev_actor[N:] = self.to_act[self.parent[N:]]
        sd = torch.where(t["street"].long() == 4)[0]
        self.sd_idx = sd
        self.sd_potential = t["showdown_potential"].long()[sd]
        root_of = torch.arange(M)
        for d in range(self.depth):
            a, b = self.offs[d + 1], self.offs[d + 2]
            root_of[a:b] = root_of[self.parent[a:b]]
        self.root_of = root_of
        self.boards = np.asarray(tree["boards"])
        self.sd_boards = self.boards[root_of[sd].numpy()]

        allowed_root = torch.from_numpy(cards.allowed_mask(self.boards))
        prob_root = allowed_root.float()
        prob_root = prob_root / prob_root.sum(-1, keepdim=True).clamp(min=1.0)
        self.allowed = allowed_root[root_of]
        self.allowed_prob = prob_root[root_of]

        z = lambda *s: torch.zeros(*s, dtype=torch.float32)  # noqa: E731
        self.policy = z(M, H)
        self.policy_avg = z(M, H)
        self.regrets = z(M, H)
        self.weight_sums = z(M, H)
        self.uniform = z(M, H)
        self.uniform[N:] = (1.0 / self._fan_out(self.child_count))[:, None].expand(-1, H)
        self.beliefs = z(M, 2, H)
        self.beliefs[:N] = root_beliefs.float()
        self.beliefs_avg = self.beliefs.clone()
        self.reach = z(M, 2, H)
        self.reach[:N] = 1.0
        self.reach_avg = self.reach.clone()
        self.values = z(M, 2, H)
        fold = (self.action == 0) & self.done
        self.values[fold, 0] = self.fold_value[fold][:, None]
        self.values[fold, 1] = -self.fold_value[fold][:, None]
        self.values_avg = self.values.clone()
        self.stats = {}  # `cfr_delta.*`, filled while solving

    # ---- tree primitives (sparse_cfr_evaluator.py:428-538) ----
    def _fan_out(self, x, level=None):
        if level is None:
            a, b, size = 0, self.top, self.M - self.N
        else:
            a, b = self.offs[level], self.offs[level + 1]
            size = self.offs[level + 2] - b
        return x[a:b].repeat_interleave(self.child_count[a:b], dim=0, output_size=size)

    def _pull_back_sum(self, x, out, level=None):
        a, b = (self.N, self.M) if level is None else (self.offs[level + 1], self.offs[level + 2])
        src = x[a:b] if x.shape[0] == self.M else x
        idx = self.parent[a:b][(...,) + (None,) * (src.dim() - 1)].expand(-1, *src.shape[1:])
        out.scatter_reduce_(0, idx, src, reduce="sum", include_self=True)

    def _pull_back(self, x, level=None):
        if level is None:
            pa, pb, ca, cb = 0, self.top, self.N, self.M
        else:
            pa, pb = self.offs[level], self.offs[level + 1]
            ca, cb = self.offs[level + 1], self.offs[level + 2]
        out = torch.zeros((pb - pa, self.A, *x.shape[1:]), dtype=x.dtype)
        out[self.parent[ca:cb] - pa, self.action[ca:cb]] = x[ca:cb]
        return out

    def _fan_out_deep(self, x):
        out = torch.zeros((self.M, *x.shape[1:]), dtype=x.dtype)
        out[: self.N] = x
        for d in range(self.depth):
            out[self.offs[d + 1]: self.offs[d + 2]] = self._fan_out(out, d)
        return out

    # ---- beliefs and reach (cfr_evaluator.py:248-273, 332-380) ----
    def _block(self, target):
        target.masked_fill_((~self.allowed)[:, None, :], 0.0)

    def _normalize(self, target):
        denom = target.sum(dim=-1, keepdim=True)
        torch.where(denom > 1e-5, target / denom, self.allowed_prob[:, None, :], out=target)

    def _reach_weights(self, target, policy):
        for d in range(self.depth):
            a, b = self.offs[d + 1], self.offs[d + 2]
            dest = target[a:b]
            dest[:] = self._fan_out(target, level=d)
            idx = self.prev_actor[a:b][:, None, None].expand(-1, -1, H)
            dest.scatter_reduce_(1, idx, policy[a:b][:, None], reduce="prod", include_self=True)
        self._block(target)

    def _propagate_beliefs(self, target, reach):
        target[:] = self._fan_out_deep(target[: self.N]) * reach
        self._normalize(target)

    # ---- start of evaluate_cfr (cfr_evaluator.py:1503-1513) ----
    def initialize(self):
        self.policy.zero_()
        for d in range(self.depth):
            a, b, c = self.offs[d], self.offs[d + 1], self.offs[d + 2]
            self.policy[b:c] = self.uniform[b:c] if self.start_policy is None else self.start_policy[b:c]
            self.beliefs[b:c] = self._fan_out(self.beliefs, level=d)
            rows = torch.arange(b, c)
            self.beliefs[rows, self.prev_actor[b:c]] *= self.policy[b:c]
            self._block(self.beliefs)
            self._normalize(self.beliefs)
        if self.depth == 0:
            self._block(self.beliefs)
            self._normalize(self.beliefs)
        self._reach_weights(self.reach, self.policy)
        self.policy_avg[:] = self.policy
        self.reach_avg[:] = self.reach
        self.beliefs_avg[:] = self.beliefs
        self.set_leaf_values()
        self.expected_values()
        self.values_avg[:] = self.values

    # ---- leaves and backup ----
    def set_leaf_values(self, t=0, beliefs=None):
        if beliefs is None:
            beliefs = self.beliefs_avg if self.cfr_avg else self.beliefs
        if self.model_idx.numel() and self.leaf_fn is not None:
            b = beliefs[self.model_idx]
            hv = self.leaf_fn(b, self.model_idx).float()
            if not self.cfr_avg or t <= 1 or self.last_model_values is None:
                self.values[self.model_idx] = hv
            else:  # the model's output is the average over the iterations so far: recover this iteration's
                old, new = self.mixing_weights(t)
                unmixed = (old + new) * hv - old * self.last_model_values
                unmixed /= new
                if self.enforce_zero_sum:
                    unmixed = unmixed - (unmixed * b).sum(dim=2, keepdim=True).mean(dim=1, keepdim=True)
                self.values[self.model_idx] = unmixed
            self.last_model_values = hv.clone()
        if self.sd_idx.numel():
            vals = showdown.showdown_values(self.sd_boards, beliefs[self.sd_idx], self.sd_potential,
                                            self.scale[self.sd_idx])
            self.values[self.sd_idx] = vals

    def expected_values(self, policy=None, beliefs=None, leaf_values=None, values=None):
        policy = self.policy if policy is None else policy
        beliefs = self.beliefs if beliefs is None else beliefs
        leaf_values = self.values if leaf_values is None else leaf_values
        values = leaf_values if values is None else values
        if leaf_values is values:
            values.masked_fill_((~self.leaf)[:, None, None], 0.0)
        else:
            torch.where(self.leaf[:, None, None], leaf_values, torch.zeros_like(values), out=values)
        N, top = self.N, self.top
        actor = self.to_act[:top, None, None].expand(-1, -1, H)
        actor_beliefs = beliefs[:top].gather(1, actor).squeeze(1)
        dest = self._fan_out(actor_beliefs)
        marginal = dest * policy[N:]
        blocked = unblocked.unblocked_mass(marginal)
        matchup = unblocked.unblocked_mass(dest)
        opp_policy = torch.zeros_like(policy)
        torch.where(matchup > 1e-5, blocked / matchup, torch.zeros_like(blocked), out=opp_policy[N:])
        for d in range(self.depth - 1, -1, -1):
            b, c = self.offs[d + 1], self.offs[d + 2]
            rows = torch.arange(c - b)
            pa = self.prev_actor[b:c]
            weighted = values[b:c].clone()
            weighted[rows, pa, :] *= policy[b:c]
            weighted[rows, 1 - pa, :] *= opp_policy[b:c]
            self._pull_back_sum(weighted, values, level=d)

    # ---- one iteration (cfr_evaluator.py:1331-1381) ----
    def instantaneous_regrets(self, achieved=None, expected=None):
        """`compute_instantaneous_regrets` (cfr_evaluator.py:1117-1165): values achieved by each child against the
        values expected at its parent (both the latest values unless given)."""
        N = self.N
        achieved = self.values if achieved is None else achieved
        expected = self.values if expected is None else expected
        out = torch.zeros_like(self.policy)
        actor = self.to_act[:, None, None].expand(-1, -1, H)
        pa = self.prev_actor[N:, None, None].expand(-1, -1, H)
        beliefs = self.beliefs_avg if self.cfr_avg else self.beliefs
        opp_reach = unblocked.unblocked_mass(beliefs.flip(dims=[1]))
        weights = self._fan_out(opp_reach.gather(1, actor).squeeze(1))
        exp = self._fan_out(expected.gather(1, actor).squeeze(1))
        ach = achieved[N:].gather(1, pa).squeeze(1)
        out[N:] = weights * (ach - exp)
        return out

    def mixing_weights(self, t):
        if self.cfr_type == "standard":
            return t, 1
        if self.cfr_type == "linear":
            return t, 2
        if self.cfr_type == "discounted":
            return t ** self.gamma, (t + 1) ** self.gamma
        if t > self.dcfr_delay:  # discounted_plus
            return t - self.dcfr_delay, 2
        return 0, 1

    def update_average_policy(self, t):
        if self.cfr_type in ("discounted", "discounted_plus") and t <= self.dcfr_delay:
            self.policy_avg[:] = self.policy
            return
        if t == 0:
            self.policy_avg[:] = self.policy
            return
        N, top = self.N, self.top
        old, new = self.mixing_weights(t)
        actor = self.to_act[:top, None, None].expand(-1, -1, H)
        r_new = self.reach[:top].gather(1, actor).squeeze(1)
        r_old = self.reach_avg[:top].gather(1, actor).squeeze(1)
        r_old *= old
        r_new *= new
        r_new_c = self._fan_out(r_new)
        r_old_c = self._fan_out(r_old)
        numer = r_old_c * self.policy_avg[N:] + r_new_c * self.policy[N:]
        denom = r_old_c + r_new_c
        plain = (old * self.policy_avg[N:] + new * self.policy[N:]) / (old + new)
        torch.where(denom > 1e-5, numer / denom, plain, out=self.policy_avg[N:])
        sums = torch.zeros(top, H)
        self._pull_back_sum(self.policy_avg, sums)
        pd = self._fan_out(sums)
        torch.where(pd > 1e-5, self.policy_avg[N:] / pd, self.policy_avg[N:], out=self.policy_avg[N:])
        self.policy_avg[:N] = 0.0

    def update_policy(self, t):
        N = self.N
        pos = self.regrets.clamp(min=0.0)
        sums = torch.zeros_like(self.policy)
        self._pull_back_sum(pos, sums)
        denom = self._fan_out(sums)
        torch.where(denom > 1e-8, pos[N:] / denom.clamp(min=1e-8), self.uniform[N:], out=self.policy[N:])
        self._reach_weights(self.reach, self.policy)
        self._propagate_beliefs(self.beliefs, self.reach)
        self.update_average_policy(t)
        self._reach_weights(self.reach_avg, self.policy_avg)
        self._propagate_beliefs(self.beliefs_avg, self.reach_avg)

    def apply_schedules(self, t):
        total = max(1, self.iterations - self.warm_start_iterations)
        progress = min(1.0, max(0.0, max(0, t - self.warm_start_iterations) / float(total)))
        for name in ("alpha", "beta", "gamma"):
            first, last = getattr(self, name + "0"), getattr(self, name + "_final")
            setattr(self, name, first if last is None else first + (last - first) * progress)

    def iteration(self, t):
        self.apply_schedules(t)
        inst = self.instantaneous_regrets()
        if self.cfr_type == "linear":
            inst.masked_fill_(self.prev_actor[:, None] == t % 2, 0.0)
        elif self.cfr_type in ("discounted", "discounted_plus"):
            pos = self.regrets > 0
            num = torch.where(pos, t ** self.alpha, t ** self.beta)
            den = torch.where(pos, t ** self.alpha + 1, t ** self.beta + 1)
            self.regrets *= num
            self.regrets /= den
            self.weight_sums *= num
            self.weight_sums /= den
        self.weight_sums += 1
        self.regrets += inst
        if self.cfr_plus:
            self.regrets.clamp_(min=0)
        before = self.policy.clone()
        self.update_policy(t)
        self.record_policy_delta(t, before)
        self.set_leaf_values(t)
        self.expected_values()
        if not self.final_policy_values:
            self.update_average_values(t)

    def record_policy_delta(self, t, before):
        """`_record_stats` (cfr_evaluator.py:1573-1605): at the iterations linspace(warm start, T - 1, 5), the
        absolute change of the policy summed over actions and reachable hands, per reachable hand, averaged
        over the nodes some hand reaches (all nodes above the deepest level).  Where two of the five points
        fall on one iteration the first one names the key."""
        points = torch.linspace(self.warm_start_iterations, self.iterations - 1, 5).round().int().tolist()
        if t not in points:
            return
        percentile = (0, 25, 50, 75, 100)[points.index(t)]
        diff = self._pull_back(self.policy) - self._pull_back(before)
        reachable = (self.reach > 0).any(dim=1)[: self.top]
        diff.masked_fill_(~reachable[:, None, :], 0.0)
        count = reachable.sum(dim=-1)
        nodes = count > 0
        total = diff.abs().sum(dim=1).sum(dim=1)
        delta = torch.where(nodes, total / count, 0.0)
        self.stats[f"cfr_delta.{percentile}"] = (delta.sum() / nodes.sum()).item()

    def _zero_sum(self, values, beliefs):
        sums = (values * beliefs).sum(dim=2, keepdim=True).mean(dim=1, keepdim=True)
        sums.masked_fill_(self.done[:, None, None], 0.0)
        return values - sums

    def update_average_values(self, t):
        """cfr_evaluator.py:1260-1274."""
        old, new = self.mixing_weights(t)
        self.values_avg *= old
        self.values_avg += new * self.values
        self.values_avg /= old + new
        if self.enforce_zero_sum:
            self.values_avg = self._zero_sum(self.values_avg, self.beliefs_avg)

    def finalize(self):
        """update_average_values_final (cfr_evaluator.py:1276-1292)."""
        self.set_leaf_values(0, beliefs=self.beliefs_avg)
        self.expected_values(self.policy_avg, self.beliefs_avg, self.values, self.values_avg)
        if self.enforce_zero_sum:
            sums = (self.values_avg * self.beliefs_avg).sum(dim=2, keepdim=True).mean(dim=1, keepdim=True)
            sums.masked_fill_(self.done[:, None, None], 0.0)
            self.values_avg = self.values_avg - sums

    def warm_start(self):
        """Type `model` (cfr_evaluator.py:913-926): cumulative regrets = start policy x weight,
        weight = iterations x multiplier x mean positive instantaneous regret of the row.
        Type `model_br` (:927-955): cumulative regrets = iterations x multiplier x the regrets of not playing
        a best response against the start policy."""
        N, ws = self.N, self.warm_start_iterations
        weight = float(ws) * float(self.warm_start_multiplier)
        if self.warm_start_type == "model":
            regrets = self.instantaneous_regrets()
            weights = weight * regrets[N:].clamp(min=0.0).mean(dim=-1)
            self.regrets[N:] = self.policy[N:] * weights[:, None]
            self.weight_sums[N:] = weights[:, None]
        else:
            br = [self._best_response(self.policy, self.beliefs, self.values, torch.full((self.M,), pl, dtype=torch.long))
                  for pl in range(2)]
            values_br = torch.where(self.prev_actor[:, None, None] == 0, br[0], br[1])
            self.regrets += weight * self.instantaneous_regrets(values_br, self.values)
            self.weight_sums += weight
        self.update_policy(ws)
        self.set_leaf_values()
        self.expected_values()
        self.values_avg[:] = self.values

    def solve(self):
        self.initialize()
        if self.warm_start_iterations > 0:
            self.warm_start()
        for t in range(self.warm_start_iterations, self.iterations):
            self.iteration(t)
        if self.final_policy_values:
            self.finalize()
        return self

    # ---- local exploitability of the average policy (cfr_evaluator.py:603-764) ----
    def _best_response(self, policy, beliefs, base_values, deviator):
        top, A = self.top, self.A
        vbr = torch.where(self.leaf[:, None, None], base_values, torch.zeros(()))
        minv = torch.finfo(torch.float32).min
        pol_src = self._pull_back(policy)
        actor_all = self.to_act[:, None, None].expand(-1, -1, H)
        actor_beliefs = beliefs.gather(1, actor_all).squeeze(1)[:top]
        matchup = unblocked.unblocked_mass(actor_beliefs)
        pol_blocked = unblocked.unblocked_mass(pol_src * actor_beliefs[:, None, :])
        opp_pol = torch.where(matchup[:, None, :] > 1e-5, pol_blocked / matchup[:, None, :], torch.zeros(()))
        child_mask = pol_src.new_zeros((top, A), dtype=torch.bool)
        child_mask[self.parent[self.N:], self.action[self.N:]] = True
        for d in range(self.depth - 1, -1, -1):
            a, b = self.offs[d], self.offs[d + 1]
            rows = torch.arange(b - a)
            actor = self.to_act[a:b]
            dev = deviator[a:b]
            vsrc = self._pull_back(vbr, level=d)  # [K,A,2,H]
            ai = actor[:, None, None, None].expand(-1, A, 1, H)
            av = vsrc.gather(2, ai).squeeze(2)
            ov = vsrc.gather(2, 1 - ai).squeeze(2)
            best = av.masked_fill(~child_mask[a:b][:, :, None], minv).argmax(dim=1)
            best_v = av.gather(1, best[:, None, :]).squeeze(1)
            db = actor_beliefs[a:b]
            mass = torch.zeros(b - a, A, H)
            mass.scatter_add_(1, best[:, None, :], db[:, None, :])
            mb = unblocked.unblocked_mass(mass)
            dm = matchup[a:b][:, None, :]
            p_dev = torch.where(dm > 1e-5, mb / dm, torch.zeros(()))
            v_opp = (p_dev * ov).sum(dim=1)
            is_dev = (dev == actor)[:, None]
            actor_values = torch.where(is_dev, best_v, (av * pol_src[a:b]).sum(dim=1))
            opp_values = torch.where(is_dev, v_opp, (ov * opp_pol[a:b]).sum(dim=1))
            vbr[rows + a, actor] = actor_values
            vbr[rows + a, 1 - actor] = opp_values
            torch.where(self.leaf[a:b, None, None], base_values[a:b], vbr[a:b], out=vbr[a:b])
        return vbr

    def exploitability(self):
        N = self.N
        leaf_values = self.values_avg.clamp(-1.0, 1.0)
        base = torch.zeros_like(leaf_values)
        self.expected_values(self.policy_avg, self.beliefs_avg, leaf_values, base)
        gains, br_vals = [], []
        for player in range(2):
            dev = torch.full((self.M,), player, dtype=torch.long)
            br = self._best_response(self.policy_avg, self.beliefs_avg, leaf_values, dev)
            rb = self.beliefs_avg[:N, player]
            gains.append(((br[:N, player] - base[:N, player]) * rb).sum(dim=-1))
            br_vals.append((br[:N, player] * rb).sum(dim=-1))
        total = gains[0] + gains[1]
        return total, torch.stack(br_vals, dim=-1)

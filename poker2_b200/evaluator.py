"""Evaluator facade with the method names the upstream data generator calls
(`RebelDataGenerator.generate_data`, p2/search/rebel_data_generator.py:52-96):
`initialize_subgame(src_env, src_indices, initial_beliefs)`, `evaluate_cfr(training_mode)`,
`training_data(exclude_start)`; attributes `root_nodes`, `num_players`, `device`, `stats`,
`cfr_iterations` (the trainer's schedule may change it between subgames).

`src_env` is read by attribute, as the upstream `HUNLTensorEnv` exposes them (tensors or
arrays indexed by environment): board_indices [E,5] (-1 = not dealt), pot, stacks [E,2],
starting_stacks [E,2], committed [E,2], to_act, button, street, actions_this_round,
min_raise, is_allin [E,2], done, scale.  Upstream classes are not imported: the returned
batches are plain dataclasses with the fields of `RebelBatch` that do not depend on a
feature encoder (the `beliefs` member is what `features.beliefs` holds upstream).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from types import SimpleNamespace

import numpy as np
import torch

from . import leaf_eval, sampling, solver as psolver, tree as ptree

NUM_HANDS = 1326


def _np(x, dtype=None) -> np.ndarray:
    a = x.detach().cpu().numpy() if torch.is_tensor(x) else np.asarray(x)
    return a.astype(dtype) if dtype is not None else a


@dataclass
class Batch:
    """Counterpart of the upstream `RebelBatch` (p2/models/mlp/rebel_replay.py)."""

    beliefs: torch.Tensor  # [n, 2*1326] beliefs under the average policy (features.beliefs upstream)
    legal_masks: torch.Tensor  # [n, A] bool
    statistics: dict
    value_targets: torch.Tensor | None = None  # [n, 2, 1326]
    policy_targets: torch.Tensor | None = None  # [n, 1326, A]

    def __len__(self) -> int:
        return int(self.beliefs.shape[0])

    def __getitem__(self, index) -> "Batch":
        pick = lambda t: None if t is None else t[index]  # noqa: E731
        return Batch(self.beliefs[index], self.legal_masks[index], {k: v[index] for k, v in self.statistics.items()},
                     pick(self.value_targets), pick(self.policy_targets))


@dataclass
class SampledStates:
    """What `evaluate_cfr` returns: the public states the next subgames start from (upstream:
    a `PublicBeliefState`), as tree node indices, their beliefs and their betting state."""

    nodes: torch.Tensor  # [n] upstream node indices inside the solved trees
    beliefs: torch.Tensor  # [n, 2, 1326]
    state: ptree.RoundState
    boards: np.ndarray  # [n, 5]
    all_nodes: torch.Tensor = field(default=None)  # [N] the node every root's walk ended at


class SubgameEvaluator:
    num_players = 2

    def __init__(self, device, *, iterations: int, bet_bins=(0.5, 1.0), max_depth: int = 8, bb: int = 2,
                 cfr_type: str = "discounted", alpha: float = 1.5, beta: float = 0.0, gamma: float = 2.0,
                 dcfr_delay: int = 0, cfr_plus: bool = False, max_raises=None, model=None,
                 chance_average: bool = True, leaf_chunk: int = 2048, sample_epsilon: float = 0.25,
                 generator: torch.Generator | None = None, warm_start_iterations: int = 0,
                 warm_start_multiplier: float = 1.0, alpha_final: float | None = None,
                 beta_final: float | None = None, gamma_final: float | None = None,
                 enforce_zero_sum: bool = False, cfr_avg: bool = False, running_values: bool = False,
                 warm_start_type: str = "model", policy_delta_stats: bool = False):
        self.device = torch.device(device)
        self.cfr_iterations = int(iterations)
        self.bet_bins, self.max_depth, self.bb, self.max_raises = list(bet_bins), max_depth, bb, max_raises
        self.cfr_type, self.alpha, self.beta, self.gamma = cfr_type, alpha, beta, gamma
        self.dcfr_delay, self.cfr_plus = dcfr_delay, cfr_plus
        # exponent schedules (`apply_schedules`, cfr_evaluator.py:1294-1329) and the zero-sum shift of the
        # value targets upstream applies when `model.enforce_zero_sum` is set (:957-980, 1289-1292)
        self.alpha_final, self.beta_final, self.gamma_final = alpha_final, beta_final, gamma_final
        self.enforce_zero_sum = bool(enforce_zero_sum)
        # `cfr_avg` upstream: leaf values and regret weights at the beliefs under the average policy, model
        # values de-averaged (cfr_evaluator.py:997-1018, :1029, :1133)
        self.cfr_avg = bool(cfr_avg)
        # `value_targets_from_final_policy = False` upstream: value targets from the running average of the
        # per-iteration values (`update_average_values`, :1260-1274); solved pass by pass
        self.running_values = bool(running_values)
        self.model, self.chance_average, self.leaf_chunk = model, chance_average, leaf_chunk
        self.sample_epsilon = sample_epsilon
        self.generator = generator
        # warm start of type `model`: regrets seeded from the start policy (cfr_evaluator.py:887-926)
        self.warm_start_iterations = int(warm_start_iterations)
        self.warm_start_multiplier = float(warm_start_multiplier)
        self.warm_start_type = warm_start_type  # "model" (:913-926) or "model_br" (:927-955)
        # `cfr_delta.*` in `stats` (`_record_stats`, :1573-1605): needs the regrets on both sides of five
        # iterations, so such a solve runs pass by pass
        self.policy_delta_stats = bool(policy_delta_stats)
        self.stats: dict = {}
        self.root_nodes = 0
        self._result = None

    # ------------------------------------------------------------------ initialize_subgame
    def initialize_subgame(self, src_env, src_indices, initial_beliefs=None) -> None:
        """Builds the public trees below the given root states and the device buffers of the
        solve (cfr_evaluator.py:770-828, sparse_cfr_evaluator.py:141-306)."""
        idx = _np(src_indices, np.int64)
        take = lambda name, dt: _np(getattr(src_env, name))[idx].astype(dt)  # noqa: E731
        n = idx.shape[0]
        raises = take("raises", np.int64) if hasattr(src_env, "raises") else np.zeros(n, dtype=np.int64)
        roots = ptree.RoundState(
            to_act=take("to_act", np.int64), pot=take("pot", np.int64), stacks=take("stacks", np.int64),
            committed=take("committed", np.int64), min_raise=take("min_raise", np.int64),
            actions_this_round=take("actions_this_round", np.int64), is_allin=take("is_allin", bool),
            done=take("done", bool), street=take("street", np.int64), button=take("button", np.int64),
            starting_stacks=take("starting_stacks", np.int64), scale=take("scale", np.float32), raises=raises)
        self.boards = take("board_indices", np.int64)
        if hasattr(src_env, "last_board_indices"):
            self.last_boards = take("last_board_indices", np.int64)
        else:  # the board before the last deal: the flop comes as three cards, turn and river as one
            self.last_boards = self.boards.copy()
            n_cards = (self.boards >= 0).sum(axis=1)
            self.last_boards[n_cards == 3] = -1
            later = n_cards > 3
            self.last_boards[np.nonzero(later)[0], n_cards[later] - 1] = -1
        self.trees = ptree.build_trees(roots, self.bet_bins, self.max_depth, bb=self.bb, max_raises=self.max_raises)
        self.layout = psolver.device_layout(self.trees, self.boards)
        self.root_nodes = n
        boards_t = torch.from_numpy(self.boards)
        kw = dict(exploitability=True, keep_node_values=True, sampling=True)
        # pass by pass only where something happens between the passes: leaves valued by the network, running
        # value averages, the best-response pass of a `model_br` warm start; a warm start of type `model` and a
        # start policy fit the one-call solve, whose iteration passes run in the lean kernel
        self.stepped = (bool(self.layout.num_model_leaves) or self.running_values or self.policy_delta_stats
                        or (self.warm_start_iterations > 0 and self.warm_start_type == "model_br"))
        if self.layout.num_model_leaves:
            if self.model is None:
                raise ValueError("the subgames have non-terminal leaves: a leaf model is required")
            self.solver = psolver.SteppedSolver(self.layout, boards_t, self.device, **kw)
            leaf_boards = torch.from_numpy(self.boards[self.trees.root_of[self.layout.model_nodes]])
            ctx = leaf_eval.leaf_context(self.trees, self.layout.model_nodes)
            cls = leaf_eval.ChanceLeafEvaluator if self.chance_average else leaf_eval.DirectLeafEvaluator
            extra = dict(chunk=self.leaf_chunk) if self.chance_average else {}
            self.leaf_fn = cls(self.model, leaf_boards, ctx, self.device, **extra)
        else:
            cls = psolver.SteppedSolver if self.stepped else psolver.SubgameSolver
            self.solver = cls(self.layout, boards_t, self.device, **kw)
            self.leaf_fn = None
        self._policy_delta = None
        if self.policy_delta_stats:
            from . import stats as pstats

            self._policy_delta = pstats.PolicyDelta(self.trees, self.boards, self.layout, self.device)
        if initial_beliefs is None:
            initial_beliefs = torch.full((n, 2, NUM_HANDS), 1.0 / NUM_HANDS, dtype=torch.float32)
        self.root_beliefs = psolver.pad_rows(initial_beliefs.to(device=self.device, dtype=torch.float32)).contiguous()
        self._result = None
        self.stats["evaluator_street"] = float(roots.street.mean())
        self.stats["evaluator_total_nodes"] = float(self.trees.total_nodes)
        self.stats["evaluator_root_nodes"] = float(n)
        self.stats["evaluator_tree_depth"] = float(self.trees.tree_depth)

    # ------------------------------------------------------------------ evaluate_cfr
    def evaluate_cfr(self, training_mode: bool = True, start_policy: torch.Tensor | None = None) -> SampledStates:
        """Runs the solve (cfr_evaluator.py:1497-1528) and samples the next public states.
        start_policy [M,1326] (upstream node order): the policy head's softmax at every node;
        None = uniform, what a head with zero logits gives."""
        T, ws = self.cfr_iterations, self.warm_start_iterations
        gen_device = self.generator.device if self.generator is not None else torch.device("cpu")
        t_sample = sampling.sampling_schedule(self.root_nodes, T, self.generator, cfr_type=self.cfr_type,
                                              warm_start_iterations=ws, dcfr_delay=self.dcfr_delay, device=gen_device)
        self.t_sample = t_sample
        self.solver.set_sampling_schedule(t_sample.to(self.device), warm_start_iterations=ws)
        scal = psolver.iteration_scalars(T, cfr_type=self.cfr_type, alpha=self.alpha, beta=self.beta,
                                         gamma=self.gamma, dcfr_delay=self.dcfr_delay, alpha_final=self.alpha_final,
                                         beta_final=self.beta_final, gamma_final=self.gamma_final,
                                         warm_start_iterations=ws)
        if ws > 0 and start_policy is None:  # uniform over the children of every parent
            cc = torch.from_numpy(self.trees.child_count[self.trees.parent_index.clip(min=0)]).clamp(min=1)
            start_policy = (1.0 / cc.to(torch.float32))[:, None].expand(-1, NUM_HANDS).contiguous()
        first = None
        if ws > 0:
            first = psolver.warm_start_mix_scalars(scal, cfr_type=self.cfr_type, gamma=self.gamma,
                                                   dcfr_delay=self.dcfr_delay, warm_start_iterations=ws)
        if self.stepped:
            res = self.solver.solve(self.root_beliefs, scal, self.leaf_fn, cfr_plus=self.cfr_plus,
                                    enforce_zero_sum=self.enforce_zero_sum, start_policy=start_policy,
                                    warm_start_iterations=ws, warm_start_multiplier=self.warm_start_multiplier,
                                    warm_start_scalars=first, cfr_avg=self.cfr_avg, running_values=self.running_values,
                                    warm_start_type=self.warm_start_type, policy_delta=self._policy_delta)
        else:
            res = self.solver.solve(self.root_beliefs, scal, cfr_plus=self.cfr_plus,
                                    enforce_zero_sum=self.enforce_zero_sum, cfr_avg=self.cfr_avg,
                                    start_policy=start_policy, warm_start_iterations=ws,
                                    warm_start_multiplier=self.warm_start_multiplier, warm_start_scalars=first)
        self._result = res
        from . import stats as pstats

        self.stats.update(pstats.evaluator_stats(res, self.trees, self.boards))
        if self._policy_delta is not None and self.solver.policy_deltas:
            keys = sorted(self.solver.policy_deltas)
            vals = torch.stack([self.solver.policy_deltas[q] for q in keys]).cpu().tolist()  # one read
            self.stats.update({f"cfr_delta.{q}": v for q, v in zip(keys, vals)})
        # the walk draws from the generator: run it where the generator lives
        pol = res.level_major(res.policy_sample).to(gen_device)
        bel = res.level_major(res.beliefs_last).to(gen_device)
        nodes, cont, cont_beliefs = sampling.sample_leaves(self.trees, pol, bel, self.generator,
                                                           sample_epsilon=self.sample_epsilon,
                                                           training_mode=training_mode)
        cont_np = cont.cpu().numpy()
        return SampledStates(nodes=cont, beliefs=cont_beliefs, state=self.trees.state.take(cont_np),
                             boards=self.boards[self.trees.root_of[cont_np]], all_nodes=nodes)

    # ------------------------------------------------------------------ start policy from a policy head
    def start_policy_from_head(self, logits_fn) -> torch.Tensor:
        """The level-by-level start of `initialize_policy_and_beliefs` (cfr_evaluator.py:832-886): a policy head
        that reads the node beliefs gives the policy of one tree level at a time, because the beliefs of a level
        follow from the policies of the levels above.  For every level,
        `logits_fn(nodes [K] int64 upstream node indices, beliefs [K,2,1326] fp32) -> [K,1326,A]` policy logits;
        they are masked by the legal actions (the lowest finite value, :306-330), soft-maxed and pushed down to
        the children; the children's beliefs are the parent's, times the policy for the player who acted,
        and every row is blocked by its board and re-normalised once per level, as upstream does.
        Returns the start policy [M,1326] in the upstream node order, to hand to `evaluate_cfr`."""
        t, dev = self.trees, self.device
        offs, M, N, A = t.depth_offsets, t.total_nodes, t.num_roots, t.num_actions
        as_t = lambda a, dt=None: torch.from_numpy(np.ascontiguousarray(a)).to(dev, dt)  # noqa: E731
        parent, action, to_act = as_t(t.parent_index, torch.int64), as_t(t.action_from_parent, torch.int64), as_t(t.state.to_act, torch.int64)
        legal, child_count = as_t(t.legal_mask, torch.bool), as_t(t.child_count, torch.int64)
        root_of = as_t(t.root_of, torch.int64)
        c1, c2 = np.triu_indices(52, k=1)  # the 1326 combos in their order: (c1 < c2), c1-major
        hit = torch.zeros(N, 53, dtype=torch.bool, device=dev)
        cards = torch.from_numpy(self.boards).to(dev)
        hit.scatter_(1, torch.where(cards >= 0, cards, torch.full_like(cards, 52)), True)
        allowed_root = ~(hit[:, as_t(c1, torch.int64)] | hit[:, as_t(c2, torch.int64)])  # combos off the board
        prob_root = allowed_root.to(torch.float32)
        prob_root = prob_root / prob_root.sum(-1, keepdim=True).clamp(min=1.0)
        allowed, allowed_prob = allowed_root[root_of], prob_root[root_of]
        beliefs = torch.zeros(M, 2, NUM_HANDS, device=dev, dtype=torch.float32)
        beliefs[:N] = self.root_beliefs[..., :NUM_HANDS]
        policy = torch.zeros(M, NUM_HANDS, device=dev, dtype=torch.float32)
        for d in range(t.tree_depth):
            a, b, c = int(offs[d]), int(offs[d + 1]), int(offs[d + 2])
            logits = logits_fn(torch.arange(a, b), beliefs[a:b]).to(dev, torch.float32)
            masked = logits.masked_fill(~legal[a:b][:, None, :], torch.finfo(torch.float32).min)
            probs = torch.softmax(masked, dim=-1)
            probs.masked_fill_((child_count[a:b] == 0)[:, None, None], 0.0)
            policy[b:c] = probs[parent[b:c] - a, :, action[b:c]]
            level = beliefs[parent[b:c]].clone()
            rows = torch.arange(c - b, device=dev)
            level[rows, to_act[parent[b:c]]] *= policy[b:c]
            beliefs[b:c] = level
            beliefs.masked_fill_((~allowed)[:, None, :], 0.0)
            denom = beliefs.sum(dim=-1, keepdim=True)
            beliefs = torch.where(denom > 1e-5, beliefs / denom, allowed_prob[:, None, :].expand_as(beliefs))
        return policy

    # ------------------------------------------------------------------ state by the upstream names
    # (cfr_evaluator.py:107-170; tests and tools read these attributes).  Node order and widths are
    # the upstream ones: level-major over the batch, 1326 columns.  Available after evaluate_cfr.
    def _solved(self):
        if self._result is None:
            raise RuntimeError("call evaluate_cfr first")
        return self._result

    @property
    def policy_probs_avg(self) -> torch.Tensor:
        r = self._solved()
        return r.level_major(r.policy_avg)

    @property
    def cumulative_regrets(self) -> torch.Tensor:
        r = self._solved()
        return r.level_major(r.regrets)

    @property
    def regret_weight_sums(self) -> torch.Tensor:
        r = self._solved()
        return r.level_major(r.weight_sums)

    @property
    def policy_probs_sample(self) -> torch.Tensor:
        r = self._solved()
        return r.level_major(r.policy_sample)

    @property
    def values_avg(self) -> torch.Tensor:
        r = self._solved()
        return r.level_major(r.values_avg)

    @property
    def beliefs_avg(self) -> torch.Tensor:
        r = self._solved()
        return r.level_major(r.beliefs_avg)

    @property
    def beliefs(self) -> torch.Tensor:
        """Beliefs of the last iteration (internal nodes and model leaves; zero elsewhere)."""
        r = self._solved()
        return r.level_major(r.beliefs_last)

    @property
    def depth_offsets(self) -> list:
        return list(self.trees.depth_offsets)

    def _topology(self, name: str) -> torch.Tensor:
        return torch.from_numpy(np.ascontiguousarray(getattr(self.trees, name)))

    parent_index = property(lambda self: self._topology("parent_index"))
    action_from_parent = property(lambda self: self._topology("action_from_parent"))
    child_count = property(lambda self: self._topology("child_count"))
    child_offsets = property(lambda self: self._topology("child_offsets"))
    prev_actor = property(lambda self: self._topology("prev_actor"))
    legal_mask = property(lambda self: self._topology("legal_mask"))
    leaf_mask = property(lambda self: self._topology("leaf_mask"))

    # ------------------------------------------------------------------ training_data
    def training_data(self, exclude_start: bool = True):
        """(value batch, pre-chance value batch, policy batch) as upstream
        (cfr_evaluator.py:1384-1495).  The pre-chance batch holds, for roots at the start of the
        turn or river betting round, the expectation of the value network over the card that
        opened the street, on the beliefs held before it (:1446-1493); it needs the leaf model
        (None without one); for roots at the start of the flop round it is the expectation over
        the canonical flops and their suit orbits (`flop_chance.flop_chance_values`)."""
        if self._result is None:
            raise RuntimeError("training_data() needs evaluate_cfr() first")
        res, t = self._result, self.trees
        N, top, A = t.num_roots, t.depth_offsets[-2], t.num_actions
        dev = self.device
        pol = res.level_major(res.policy_avg)  # [M,1326]
        parent = torch.from_numpy(t.parent_index[N:]).to(dev)
        action = torch.from_numpy(t.action_from_parent[N:]).to(dev)
        by_src = torch.zeros((top, A, NUM_HANDS), dtype=torch.float32, device=dev)
        by_src[parent, action] = pol[N:]
        policy_targets = by_src.permute(0, 2, 1)
        value_targets = res.root_values[..., :NUM_HANDS].clamp(-1.0, 1.0)
        beliefs_avg = res.level_major(res.beliefs_avg)[:top].reshape(top, 2 * NUM_HANDS)
        amounts, legal = ptree.legal_bins(t.state, self.bet_bins, self.max_raises)
        st = t.state
        as_t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
        statistics = {"to_act": as_t(st.to_act), "street": as_t(st.street), "stage": as_t(2 * st.street),
                      "board": as_t(self.boards[t.root_of]), "pot": as_t(st.pot), "bet_amounts": as_t(amounts),
                      # inputs of the feature context (rebel_feature_encoder.py:96-113)
                      "button": as_t(st.button), "total_starting": as_t(st.starting_stacks.sum(axis=1).astype(np.float32)),
                      "has_bet": as_t((st.committed[:, 0] != st.committed[:, 1]) & (st.actions_this_round > 0))}
        legal_t = as_t(legal)
        value_stats = {k: v[:N] for k, v in statistics.items()}
        value_stats["local_exploitability"] = res.exploitability
        value_stats["local_best_response_values"] = res.br_values
        value_batch = Batch(beliefs_avg[:N], legal_t[:N], value_stats, value_targets=value_targets)
        if exclude_start:
            start = as_t((st.street[:N] == 0) & (st.actions_this_round[:N] == 0))
            value_batch = value_batch[~start]
        valid_top = as_t(~t.leaf_mask[:top])
        policy_batch = Batch(beliefs_avg[valid_top], legal_t[:top][valid_top],
                             {k: v[:top][valid_top] for k, v in statistics.items()},
                             policy_targets=policy_targets[valid_top])
        return value_batch, self._pre_chance_batch(value_targets, legal_t[:N], value_stats), policy_batch

    def _pre_chance_batch(self, value_targets, legal_root, value_stats):
        from . import chance

        t = self.trees
        N, st = t.num_roots, t.state
        from . import flop_chance

        single = (st.actions_this_round[:N] == 0) & ((st.street[:N] == 2) | (st.street[:N] == 3))
        flop = (st.actions_this_round[:N] == 0) & (st.street[:N] == 1)
        start = single | flop
        if self.model is None or not start.any():
            return None
        dev = self.device
        targets = value_targets.clone()
        if single.any():
            rows = torch.from_numpy(np.nonzero(single)[0]).to(dev)
            pre = self.root_beliefs[rows][..., :NUM_HANDS].contiguous()
            boards_pre = torch.from_numpy(self.last_boards[np.nonzero(single)[0]]).to(dev)
            ctx = leaf_eval.leaf_context(t, np.nonzero(single)[0]).to(dev)
            targets[rows] = chance.single_card_chance_values(
                pre, boards_pre, lambda post, samples, lookup: self.model(post, samples, ctx[lookup]))
        if flop.any():  # expectation over the three flop cards (chance_node_helper.py:218-357)
            rows = torch.from_numpy(np.nonzero(flop)[0]).to(dev)
            pre = self.root_beliefs[rows].contiguous()
            ctx = leaf_eval.leaf_context(t, np.nonzero(flop)[0]).to(dev)
            targets[rows] = flop_chance.flop_chance_values(
                pre, lambda post, boards, root: self.model(post, boards, ctx[root]), self.generator)
        stats = {k: v.clone() for k, v in value_stats.items()}
        stats["board"] = torch.from_numpy(self.last_boards[:N]).to(dev)
        street = torch.from_numpy(st.street[:N]).to(dev)
        prev = torch.where((street > 0) & (street < 4) & torch.from_numpy(st.actions_this_round[:N] == 0).to(dev),
                           street - 1, street)
        stats["street"], stats["stage"] = prev, 2 * prev + 1
        batch = Batch(self.root_beliefs[..., :NUM_HANDS].reshape(N, -1), legal_root, stats, value_targets=targets)
        return batch[torch.from_numpy(start).to(dev)]


def env_view(roots: ptree.RoundState, boards) -> SimpleNamespace:
    """An object with the attributes `initialize_subgame` reads, from a `RoundState` and the
    boards of the same rows (for callers that do not hold an upstream environment)."""
    ns = SimpleNamespace(**{k: v for k, v in roots.__dict__.items()})
    ns.board_indices = np.asarray(boards, dtype=np.int64)
    return ns

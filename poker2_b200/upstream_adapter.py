"""Drop-in evaluator for the upstream data-generation loop.

`RebelDataGenerator.generate_data` (p2/search/rebel_data_generator.py:52-95) drives an evaluator
through `initialize_subgame(pbs.env, indices, pbs.beliefs)` -> `evaluate_cfr()` -> `training_data()`
and feeds the returned public belief state into the next round.  `B200CFREvaluator` has the upstream
constructor `(model, device, cfg, generator)` (p2/search/sparse_cfr_evaluator.py:20-26), reads the
same `cfg.search.*` / `cfg.env.*` fields (:32-58), and returns objects with the attributes that loop
touches:

  * `evaluate_cfr()` -> `PublicBeliefStateLike(env, beliefs)`; `env` is an `EnvState`: every state
    tensor of the upstream `HUNLTensorEnv` (p2/env/hunl_tensor_env.py:105-168) at the sampled public
    states, `N`, `device` and `copy_state_from` (:489-563), so it can be the source of the next
    `initialize_subgame` and of the generator's `_extend_pbs` copy.
  * `training_data()` -> three `RebelBatchLike` with the fields of `RebelBatch`
    (p2/rl/rebel_batch.py:16-68): `features` (context, street, to_act, board, beliefs as the upstream
    `RebelFeatureEncoder` lays them out, p2/models/mlp/rebel_feature_encoder.py:52-137),
    `legal_masks`, `policy_targets`, `value_targets`, `statistics`, `len()`, indexing, `to`, `cat`.
  * `stats`: the evaluator statistics under the upstream keys.

No upstream module is imported.  The leaf model is called as `model(beliefs [S,2,1326], boards [S,5],
context [S,3])` (see `leaf_eval`); a model object may carry that callable as `b200_leaf_model`.
Every `cfg.search` combination of the sparse evaluator is accepted (CFR types standard, linear, discounted,
discounted_plus; `cfr_plus`, `cfr_avg`, both warm start types, value targets from the final policy or from the
running average).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from . import evaluator as pevaluator

NUM_HANDS = 1326

ENV_FIELDS = ("button", "street", "to_act", "last_to_act", "pot", "min_raise", "actions_this_round",
              "actions_last_round", "acted_since_reset", "stacks", "committed", "has_folded", "is_allin",
              "chips_placed", "starting_stacks", "scale", "board_indices", "last_board_indices", "hole_indices",
              "done", "winner", "deck", "deck_pos")
_OPTIONAL_FIELDS = ("raises",)  # per-street raise count of trees built with a raise cap (not an upstream field)


class EnvState:
    """The state tensors of a batch of public states, under the attribute names of the upstream
    environment.  Enough of its interface for the data-generation loop: `N`, `device`, attribute
    reads, `copy_state_from`."""

    def __init__(self, tensors: dict, device=None):
        first = next(iter(tensors.values()))
        self.N = int(first.shape[0])
        self.device = torch.device(device) if device is not None else first.device
        for name, value in tensors.items():
            setattr(self, name, value.to(self.device))
        self._names = tuple(tensors)

    @classmethod
    def from_env(cls, env, indices=None, device=None) -> "EnvState":
        """Copies the known state fields of an environment-like object (an upstream HUNLTensorEnv, an
        `EnvState`, a namespace of arrays); fields it lacks get their reset values."""
        idx = None if indices is None else torch.as_tensor(np.asarray(_host(indices)), dtype=torch.long)
        n = int(idx.numel()) if idx is not None else int(_host(getattr(env, "pot")).shape[0])
        out = {}
        for name in ENV_FIELDS + _OPTIONAL_FIELDS:
            if hasattr(env, name):
                t = torch.as_tensor(_host(getattr(env, name)))
                out[name] = t[idx].clone() if idx is not None else t.clone()
        for name, (shape, dtype, fill) in _defaults(n).items():
            out.setdefault(name, torch.full(shape, fill, dtype=dtype))
        return cls(out, device)

    def copy_state_from(self, src_env, src_select, dest_select, copy_deck: bool = True) -> None:
        """Rows `src_select` of `src_env` into rows `dest_select` of this state (hunl_tensor_env.py:489-563)."""
        for name in self._names:
            if not copy_deck and name in ("deck", "deck_pos"):
                continue
            if hasattr(src_env, name):
                getattr(self, name)[dest_select] = torch.as_tensor(getattr(src_env, name)).to(self.device)[src_select]


def _host(x):
    return x.detach().cpu() if torch.is_tensor(x) else np.asarray(x)


def _defaults(n: int) -> dict:
    i64, b = torch.int64, torch.bool
    return {
        "last_to_act": ((n,), i64, 0), "actions_last_round": ((n,), i64, 0), "acted_since_reset": ((n,), b, False),
        "has_folded": ((n, 2), b, False), "chips_placed": ((n, 2), i64, 0), "hole_indices": ((n, 2, 2), i64, -1),
        "winner": ((n,), i64, -1), "deck": ((n, 9), i64, 0), "deck_pos": ((n,), i64, 0),
        "last_board_indices": ((n, 5), i64, -1),
    }


@dataclass
class PublicBeliefStateLike:
    """`PublicBeliefState` of the upstream loop (cfr_evaluator.py:52-86): `env` and `beliefs`."""

    env: EnvState
    beliefs: torch.Tensor  # [n, 2, 1326]


@dataclass
class FeatureView:
    """The fields of the upstream `MLPFeatures` (p2/models/mlp/mlp_features.py:13-27)."""

    context: torch.Tensor  # [n,4]: to_act, position relative to the button, pot fraction, bet-faced flag
    street: torch.Tensor  # [n] (zeros: unused by the upstream encoder)
    to_act: torch.Tensor  # [n]
    board: torch.Tensor  # [n,5]
    beliefs: torch.Tensor  # [n, 2*1326]

    def __len__(self) -> int:
        return int(self.context.shape[0])

    def __getitem__(self, index) -> "FeatureView":
        return FeatureView(self.context[index], self.street[index], self.to_act[index], self.board[index],
                           self.beliefs[index])

    def to(self, device) -> "FeatureView":
        return FeatureView(*(t.to(device) for t in (self.context, self.street, self.to_act, self.board, self.beliefs)))

    @classmethod
    def cat(cls, items) -> "FeatureView":
        return cls(*(torch.cat([getattr(f, n) for f in items], dim=0)
                     for n in ("context", "street", "to_act", "board", "beliefs")))


@dataclass
class RebelBatchLike:
    """The fields and helpers of the upstream `RebelBatch` (p2/rl/rebel_batch.py:16-68, cat :128)."""

    features: FeatureView
    legal_masks: torch.Tensor
    policy_targets: torch.Tensor | None = None
    value_targets: torch.Tensor | None = None
    statistics: dict = field(default_factory=dict)

    def __len__(self) -> int:
        return len(self.features)

    def __getitem__(self, index) -> "RebelBatchLike":
        pick = lambda t: None if t is None else t[index]  # noqa: E731
        return RebelBatchLike(self.features[index], self.legal_masks[index], pick(self.policy_targets),
                              pick(self.value_targets), {k: v[index] for k, v in self.statistics.items()})

    def to(self, device) -> "RebelBatchLike":
        mv = lambda t: None if t is None else t.to(device)  # noqa: E731
        return RebelBatchLike(self.features.to(device), self.legal_masks.to(device), mv(self.policy_targets),
                              mv(self.value_targets), {k: v.to(device) for k, v in self.statistics.items()})

    @classmethod
    def cat(cls, batches) -> "RebelBatchLike":
        if not batches or any(b is None for b in batches):
            raise ValueError("cannot concatenate an empty list of batches or one that holds None")
        join = lambda name: (None if getattr(batches[0], name) is None  # noqa: E731
                             else torch.cat([getattr(b, name) for b in batches], dim=0))
        keys = batches[0].statistics.keys()
        return cls(FeatureView.cat([b.features for b in batches]), join("legal_masks"), join("policy_targets"),
                   join("value_targets"), {k: torch.cat([b.statistics[k] for b in batches], dim=0) for k in keys})


def _enum_name(x) -> str:
    return getattr(x, "name", str(x))


class B200CFREvaluator:
    """`SparseCFREvaluator(model, device, cfg, generator)` on the CUDA solver."""

    num_players = 2

    def __init__(self, model, device, cfg, generator: torch.Generator | None = None, *, max_raises=None,
                 policy_delta_stats: bool = False):
        """policy_delta_stats: also record `cfr_delta.*` (`_record_stats`, cfr_evaluator.py:1573-1605); such
        a solve runs pass by pass instead of through the one-call solve (upstream pays for these keys the
        same way: its graphed iteration leaves them out, fused_sparse_cfr_evaluator.py:522-527)."""
        s, e = cfg.search, cfg.env
        cfr_type = _enum_name(s.cfr_type)
        iterations = int(s.iterations)
        # same clamp as upstream (sparse_cfr_evaluator.py:39-41)
        ws = max(0, min(int(s.warm_start_iterations), max(1, iterations - 1)))
        ws_type = _enum_name(getattr(s, "warm_start_type", "model"))
        if ws > 0 and ws_type not in ("model", "model_br"):
            raise NotImplementedError(f"warm start of type {ws_type!r} is not supported")
        self.model, self.cfg = model, cfg
        self.device = torch.device(device)
        self.bet_bins = list(e.bet_bins)
        self.num_actions = len(self.bet_bins) + 3
        leaf_model = getattr(model, "b200_leaf_model", model if callable(model) else None)
        self._ev = pevaluator.SubgameEvaluator(
            self.device, iterations=iterations, bet_bins=self.bet_bins, max_depth=int(s.depth), bb=int(e.bb),
            cfr_type=cfr_type, alpha=float(s.dcfr_alpha), beta=float(s.dcfr_beta), gamma=float(s.dcfr_gamma),
            alpha_final=_opt(s, "dcfr_alpha_final"), beta_final=_opt(s, "dcfr_beta_final"),
            gamma_final=_opt(s, "dcfr_gamma_final"), dcfr_delay=int(s.dcfr_plus_delay), cfr_plus=bool(s.cfr_plus),
            max_raises=max_raises, model=leaf_model, chance_average=False,
            sample_epsilon=float(getattr(s, "sample_epsilon", 0.25)), generator=generator, warm_start_iterations=ws,
            warm_start_multiplier=float(getattr(s, "warm_start_multiplier", 1.0)),
            enforce_zero_sum=bool(getattr(model, "enforce_zero_sum", False)), cfr_avg=bool(getattr(s, "cfr_avg", False)),
            running_values=not bool(getattr(s, "value_targets_from_final_policy", True)),
            warm_start_type=ws_type if ws > 0 else "model", policy_delta_stats=policy_delta_stats)
        self.root_nodes = int(cfg.num_envs)
        self.warm_start_iterations = ws
        self.generator = generator

    @classmethod
    def from_keywords(cls, search_batch_size: int, env_proto, model, bet_bins, max_depth: int, cfr_iterations: int,
                      device, float_dtype=torch.float32, generator: torch.Generator | None = None,
                      warm_start_iterations: int = 15, warm_start_type="model_br", warm_start_multiplier: float = 1.0,
                      num_supervisions: int = 1, cfr_type="linear", cfr_avg: bool = True, cfr_plus: bool = True,
                      dcfr_alpha: float = 1.5, dcfr_beta: float = 0.0, dcfr_gamma: float = 2.0,
                      dcfr_alpha_final: float | None = None, dcfr_beta_final: float | None = None,
                      dcfr_gamma_final: float | None = None, dcfr_delay: int = 0, sample_epsilon: float = 0.25,
                      value_targets_from_final_policy: bool = False, **kw) -> "B200CFREvaluator":
        """The keyword constructor of the dense `RebelCFREvaluator` (rebel_cfr_evaluator.py:73-100), same
        argument names and defaults, on this evaluator: the solve is the same CFR on the same public tree;
        the state tensors keep the sparse node order (valid nodes only, level-major), not the dense
        A**depth layout.  `env_proto` supplies the big blind; solver state is fp32 whatever `float_dtype`
        says, and `num_supervisions` belongs to the trainer."""
        from types import SimpleNamespace

        if float_dtype not in (torch.float32, None):
            raise ValueError("the solver state is fp32")
        search = SimpleNamespace(
            depth=int(max_depth), iterations=int(cfr_iterations), warm_start_iterations=int(warm_start_iterations),
            warm_start_type=warm_start_type, warm_start_multiplier=float(warm_start_multiplier), cfr_type=cfr_type,
            cfr_avg=bool(cfr_avg), cfr_plus=bool(cfr_plus), dcfr_alpha=dcfr_alpha, dcfr_beta=dcfr_beta,
            dcfr_gamma=dcfr_gamma, dcfr_alpha_final=dcfr_alpha_final, dcfr_beta_final=dcfr_beta_final,
            dcfr_gamma_final=dcfr_gamma_final, dcfr_plus_delay=int(dcfr_delay), sample_epsilon=float(sample_epsilon),
            value_targets_from_final_policy=bool(value_targets_from_final_policy))
        env = SimpleNamespace(bet_bins=list(bet_bins), sb=int(getattr(env_proto, "sb", 1)), bb=int(getattr(env_proto, "bb", 2)))
        cfg = SimpleNamespace(search=search, env=env, num_envs=int(search_batch_size), seed=0)
        return cls(model, device, cfg, generator, **kw)

    # attributes the trainer reads or mutates (cfr_trainer.py:194-234)
    @property
    def cfr_iterations(self) -> int:
        return self._ev.cfr_iterations

    @cfr_iterations.setter
    def cfr_iterations(self, value: int) -> None:
        self._ev.cfr_iterations = int(value)

    @property
    def stats(self) -> dict:
        return self._ev.stats

    def __getattr__(self, name):  # solver state under the upstream names (policy_probs_avg, ...)
        if name.startswith("_"):
            raise AttributeError(name)
        return getattr(self._ev, name)

    def initialize_subgame(self, src_env, src_indices, initial_beliefs=None) -> None:
        self._src = EnvState.from_env(src_env, src_indices, device="cpu")
        self._ev.generator = self.generator
        self._ev.initialize_subgame(self._src, torch.arange(self._src.N), initial_beliefs)
        self.root_nodes = self._ev.root_nodes

    def evaluate_cfr(self, training_mode: bool = True, start_policy: torch.Tensor | None = None):
        sampled = self._ev.evaluate_cfr(training_mode=training_mode, start_policy=start_policy)
        return PublicBeliefStateLike(env=self._next_env(sampled), beliefs=sampled.beliefs.to(self.device))

    def _next_env(self, sampled) -> EnvState:
        """The environment state at the sampled tree nodes, every field as the upstream tree
        environment holds it there (hunl_tensor_env.py `step`, :766-992)."""
        t, src = self._ev.trees, self._src
        nodes = sampled.nodes.cpu().numpy().astype(np.int64)
        st = t.state.take(nodes)
        root = t.root_of[nodes]
        parent = t.parent_index[nodes]
        n = nodes.shape[0]
        as_t = lambda a, dt=None: torch.from_numpy(np.ascontiguousarray(a if dt is None else a.astype(dt)))  # noqa: E731
        deck = src.deck[root]
        n_cards = np.where(st.street >= 3, 5, np.where(st.street == 2, 4, np.where(st.street == 1, 3, 0)))
        slots = np.arange(5)[None, :]
        board = torch.where(as_t(slots < n_cards[:, None]), deck[:, 4:9], torch.full((n, 5), -1, dtype=torch.int64))
        src_board = src.board_indices[root]
        src_last = src.last_board_indices[root]
        new_street = st.street != t.state.street[root]
        last_board = torch.where(as_t(new_street)[:, None], src_board, src_last)
        placed = src.chips_placed[root] + (src.stacks[root] - as_t(st.stacks, np.int64))
        fields = {
            "button": as_t(st.button, np.int64), "street": as_t(st.street, np.int64), "to_act": as_t(st.to_act, np.int64),
            "last_to_act": as_t(t.state.to_act[parent], np.int64), "pot": as_t(st.pot, np.int64),
            "min_raise": as_t(st.min_raise, np.int64), "actions_this_round": as_t(st.actions_this_round, np.int64),
            "actions_last_round": torch.where(as_t(new_street), as_t(t.state.actions_this_round[parent] + 1, np.int64),
                                              src.actions_last_round[root]),
            "acted_since_reset": torch.ones(n, dtype=torch.bool),
            "stacks": as_t(st.stacks, np.int64), "committed": as_t(st.committed, np.int64),
            "has_folded": torch.zeros(n, 2, dtype=torch.bool), "is_allin": as_t(st.is_allin, bool),
            "chips_placed": placed, "starting_stacks": as_t(st.starting_stacks, np.int64),
            "scale": as_t(st.scale, np.float32), "board_indices": board, "last_board_indices": last_board,
            "hole_indices": src.hole_indices[root], "done": as_t(st.done, bool),
            "winner": torch.full((n,), -1, dtype=torch.int64), "deck": deck,
            "deck_pos": torch.from_numpy(4 + n_cards).to(torch.int64),
        }
        if hasattr(st, "raises") and st.raises is not None:
            fields["raises"] = as_t(st.raises, np.int64)
        return EnvState(fields, self.device)

    def training_data(self, exclude_start: bool = True):
        value, pre, policy = self._ev.training_data(exclude_start=exclude_start)
        return self._wrap(value, False), self._wrap(pre, True), self._wrap(policy, False)

    def _wrap(self, batch, pre_chance: bool):
        if batch is None:
            return None
        st = batch.statistics
        dev = batch.beliefs.device
        n = len(batch)
        to_act = st["to_act"]
        context = torch.zeros(n, 4, dtype=torch.float32, device=dev)
        if n:
            context[:, 0] = to_act.to(torch.float32)
            context[:, 1] = ((to_act - st["button"]) % 2).to(torch.float32)
            context[:, 2] = (st["pot"].to(torch.float32) / st["total_starting"].clamp(min=1.0)).clamp(0.0, 10.0)
            context[:, 3] = st["has_bet"].to(torch.float32)
        feats = FeatureView(context, torch.zeros(n, dtype=torch.float32, device=dev), to_act, st["board"], batch.beliefs)
        keep = {k: v for k, v in st.items() if k not in ("button", "total_starting", "has_bet")}
        return RebelBatchLike(feats, batch.legal_masks, batch.policy_targets, batch.value_targets, keep)


def _opt(obj, name):
    v = getattr(obj, name, None)
    return None if v is None else float(v)

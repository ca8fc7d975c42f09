"""Tree and CFR sections of the golden-vector generator (runs the upstream evaluator).

Imported by make_golden.py.  River subgames are set up the way the upstream tests do it
(tests/test_rebel_cfr_evaluator.py:1185-1217): force the deck, check down to the river,
then overwrite pot / stacks / starting stacks / scale.
"""
from __future__ import annotations

import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
SB, BB = 1, 2
BET_BINS = [0.5, 1.0]


def save(name: str, **arrays) -> None:
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **arrays)
    print(f"wrote {path} ({os.path.getsize(path) / 1024:.1f} KiB)")


class ZeroModel:
    """Leaf/policy model stand-in: zero logits (uniform initial policy), zero values."""

    enforce_zero_sum = False
    hidden_dim = 1

    def __init__(self, num_actions: int):
        self.num_actions = num_actions

    def eval(self):
        pass

    def create_feature_encoder(self, env, device=None, dtype=None):
        from p2.models.mlp.rebel_feature_encoder import RebelFeatureEncoder

        return RebelFeatureEncoder(env=env, device=device, dtype=dtype)

    def __call__(self, features, include_policy=True, **kw):
        from p2.models.model_output import ModelOutput

        n = len(features)
        return ModelOutput(policy_logits=torch.zeros(n, 1326, self.num_actions), value=torch.zeros(n),
                           hand_values=torch.zeros(n, 2, 1326))


def install_raise_cap(cap):
    """Adds a per-street cap on bets/raises/all-ins to the upstream environment by
    wrapping its methods (the upstream code has no such option).  cap=None removes it."""
    from p2.env.hunl_tensor_env import HUNLTensorEnv as Env

    if not hasattr(Env, "_orig"):
        Env._orig = dict(init=Env.__init__, copy=Env.copy_state_from, rep=Env.repeat_interleave,
                         step=Env.step_bins, legal=Env.legal_bins_amounts_and_mask)
    o = Env._orig

    def init(self, *a, **k):
        o["init"](self, *a, **k)
        self.raises = torch.zeros(self.N, dtype=torch.long)

    def copy(self, src_env, src_select, dest_select, copy_deck=True):
        o["copy"](self, src_env, src_select, dest_select, copy_deck)
        self.raises[dest_select] = src_env.raises[src_select]

    def rep(self, repeats, output_size):
        dst = o["rep"](self, repeats, output_size)
        dst.raises[:] = self.raises.repeat_interleave(repeats, dim=0, output_size=output_size)
        return dst

    def step(self, bin_indices, *a, **k):
        out = o["step"](self, bin_indices, *a, **k)
        self.raises += (bin_indices >= 2).long()
        self.raises[self.actions_this_round == 0] = 0
        return out

    def legal(self, bet_bins=None):
        amounts, mask = o["legal"](self, bet_bins)
        if Env._cap is not None:
            mask[:, 2:] &= (self.raises < Env._cap)[:, None]
        return amounts, mask

    Env._cap = cap
    Env.__init__, Env.copy_state_from, Env.repeat_interleave = init, copy, rep
    Env.step_bins, Env.legal_bins_amounts_and_mask = step, legal


def river_env(boards: torch.Tensor, pot: torch.Tensor, stack: torch.Tensor):
    from p2.env.hunl_tensor_env import HUNLTensorEnv

    n = boards.shape[0]
    env = HUNLTensorEnv(num_envs=n, starting_stack=1000, sb=SB, bb=BB, default_bet_bins=BET_BINS,
                        device=torch.device("cpu"), rng=torch.Generator().manual_seed(0))
    decks = []
    for b in boards.tolist():
        unused = [c for c in range(52) if c not in b]
        decks.append(unused[:4] + b)
    env.reset(force_deck=torch.tensor(decks), force_button=torch.zeros(n, dtype=torch.long))
    for _ in range(6):
        env.step_bins(torch.ones(n, dtype=torch.long))
    assert (env.street == 3).all() and (env.actions_this_round == 0).all()
    env.pot[:] = pot
    env.stacks[:] = stack[:, None]
    env.starting_stacks[:] = (stack + pot // 2)[:, None]
    env.scale[:] = (stack + pot // 2).float()
    if hasattr(env, "raises"):
        env.raises[:] = 0
    return env


def make_evaluator(n, iterations, depth=8, search=None, enforce_zero_sum=False):
    """search: overrides of cfg.search fields (name -> value), applied after the defaults below."""
    from p2.core.structured_config import CFRType, Config
    from p2.search.sparse_cfr_evaluator import SparseCFREvaluator

    cfg = Config()
    cfg.device = "cpu"
    cfg.seed = 0
    cfg.num_envs = n
    cfg.env.bet_bins = BET_BINS
    cfg.env.sb, cfg.env.bb = SB, BB
    cfg.search.depth = depth
    cfg.search.iterations = iterations
    cfg.search.warm_start_iterations = 0
    cfg.search.cfr_type = CFRType.discounted
    cfg.search.cfr_plus = False
    cfg.search.cfr_avg = False
    cfg.search.dcfr_alpha, cfg.search.dcfr_beta, cfg.search.dcfr_gamma = 1.5, 0.0, 2.0
    cfg.search.dcfr_plus_delay = 0
    cfg.search.value_targets_from_final_policy = True
    for name, value in (search or {}).items():
        assert hasattr(cfg.search, name), name
        setattr(cfg.search, name, value)
    model = ZeroModel(len(BET_BINS) + 3)
    model.enforce_zero_sum = enforce_zero_sum
    ev = SparseCFREvaluator(model, torch.device("cpu"), cfg, generator=torch.Generator().manual_seed(0))
    ev.sample_leaves = lambda training_mode: None
    return ev


def tree_arrays(ev) -> dict:
    fold = (ev.action_from_parent == 0) & ev.env.done
    potential = ev.env.stacks + ev.env.pot[:, None] - ev.env.starting_stacks
    return dict(
        depth_offsets=np.asarray(ev.depth_offsets, dtype=np.int64),
        parent_index=ev.parent_index.numpy(), action_from_parent=ev.action_from_parent.numpy(),
        to_act=ev.env.to_act.numpy(), legal_mask=ev.legal_mask.numpy(), leaf_mask=ev.leaf_mask.numpy(),
        child_count=ev.child_count.numpy(), child_offsets=ev.child_offsets.numpy(), done=ev.env.done.numpy(),
        street=ev.env.street.numpy(), pot=ev.env.pot.numpy(), stacks=ev.env.stacks.numpy(),
        fold_value=torch.where(fold, ev.latest_values[:, 0, 0], torch.zeros(())).numpy(),
        showdown_potential=potential.numpy(), scale=ev.env.scale.numpy(), prev_actor=ev.prev_actor.numpy(),
    )


def seeded_inputs(seed, n, pot_range=None, stack_range=None):
    import make_golden

    g = torch.Generator().manual_seed(seed)
    boards = torch.stack([torch.randperm(52, generator=g)[:5] for _ in range(n)])
    ranges = make_golden.dirichlet_ranges(boards, g)
    if pot_range is None:
        pot = torch.full((n,), 100, dtype=torch.long)
        stack = torch.full((n,), 400, dtype=torch.long)
    else:
        pot = torch.randint(pot_range[0], pot_range[1] + 1, (n,), generator=g)
        stack = torch.randint(stack_range[0], stack_range[1] + 1, (n,), generator=g)
    return boards, ranges, pot, stack


def gen_tree() -> None:
    """Tree indices and legal masks for a spread of pot/stack ratios, capped and uncapped."""
    pots = torch.tensor([100, 20, 200, 37, 150, 20, 199, 64, 90, 120])
    stacks = torch.tensor([400, 1000, 100, 333, 75, 100, 1000, 32, 45, 60])
    g = torch.Generator().manual_seed(5)
    boards = torch.stack([torch.randperm(52, generator=g)[:5] for _ in range(len(pots))])
    out = {}
    for tag, cap, depth in (("cap2", 2, 8), ("nocap", None, 5)):
        install_raise_cap(cap)
        ev = make_evaluator(len(pots), 1, depth=depth)
        ev.initialize_subgame(river_env(boards, pots, stacks), torch.arange(len(pots)), None)
        for k, v in tree_arrays(ev).items():
            out[f"{tag}_{k}"] = v
        out[f"{tag}_max_depth"] = np.int64(depth)
        print(tag, "nodes", ev.total_nodes, "depth", ev.tree_depth)
    install_raise_cap(None)
    save("tree.npz", pots=pots.numpy(), stacks=stacks.numpy(), **out)


def run_cfr(tag, boards, ranges, pot, stack, iterations, cap, depth=8, keep_all=False):
    install_raise_cap(cap)
    n = boards.shape[0]
    ev = make_evaluator(n, iterations, depth=depth)
    ev.initialize_subgame(river_env(boards, pot, stack), torch.arange(n), ranges)
    ev.evaluate_cfr()
    ex = ev._compute_exploitability()
    install_raise_cap(None)
    print(tag, "nodes", ev.total_nodes, "exploitability", ex.local_exploitability.tolist()[:4])
    out = dict(
        boards=boards.to(torch.int16).numpy(), ranges=ranges.numpy(), pot=pot.numpy(), stack=stack.numpy(),
        iterations=np.int64(iterations), cap=np.int64(-1 if cap is None else cap), max_depth=np.int64(depth),
        total_nodes=np.int64(ev.total_nodes),
        policy_avg=ev.policy_probs_avg.numpy(), root_values=ev.values_avg[:n].numpy(),
        exploitability=ex.local_exploitability.numpy(), br_values=ex.local_best_response_values.numpy(),
    )
    if keep_all:
        out.update(regrets=ev.cumulative_regrets.numpy(), weight_sums=ev.regret_weight_sums.numpy(),
                   policy=ev.policy_probs.numpy(), values_avg=ev.values_avg.numpy(),
                   latest_values=ev.latest_values.numpy(), beliefs=ev.beliefs.numpy())
    save(f"cfr_{tag}.npz", **out)


def gen_cfr() -> None:
    # config 0: one seeded river subgame, pot 100 / stack 400, DCFR(1.5, 0, 2), 256 iterations
    b, r, p, s = seeded_inputs(0, 1)
    run_cfr("single_cap2_t256", b, r, p, s, 256, cap=2)
    run_cfr("single_cap2_t8", b, r, p, s, 8, cap=2, keep_all=True)
    run_cfr("single_nocap_t32", b, r, p, s, 32, cap=None)
    # ragged batch: pots in [20,200], stacks in [100,1000]
    b, r, p, s = seeded_inputs(2, 4, (20, 200), (100, 1000))
    run_cfr("batch_cap2_t24", b, r, p, s, 24, cap=2)


def hand_weights() -> torch.Tensor:
    """Fixed per-hand weights in [-1, 1] used by PotEchoModel."""
    return torch.rand(1326, generator=torch.Generator().manual_seed(77)) * 2 - 1


class PotEchoModel(ZeroModel):
    """Deterministic stand-in for the value network at non-terminal leaves: the values of a
    leaf are an elementwise function of its beliefs, of a fixed per-hand weight w and of the
    pot fraction the upstream feature encoder puts into context[:, 2]
    (rebel_feature_encoder.py:104-108): s = 0.5 + pot_fraction;
    v0 = s*w + b1; v1 = (s*w)*(-0.5) + b0."""

    def __call__(self, features, include_policy=True, **kw):
        from p2.models.model_output import ModelOutput

        n = len(features)
        bel = features.beliefs.view(n, 2, 1326).float()
        s = (0.5 + features.context[:, 2].float()).view(n, 1)
        sw = s * hand_weights().view(1, 1326)
        hv = torch.stack([sw + bel[:, 1], sw * (-0.5) + bel[:, 0]], dim=1)
        return ModelOutput(policy_logits=torch.zeros(n, 1326, self.num_actions), value=torch.zeros(n), hand_values=hv)


def turn_env(boards: torch.Tensor, pot: torch.Tensor, stack: torch.Tensor):
    """Environments at the start of the turn betting round with the given 4-card boards."""
    from p2.env.hunl_tensor_env import HUNLTensorEnv

    n = boards.shape[0]
    env = HUNLTensorEnv(num_envs=n, starting_stack=1000, sb=SB, bb=BB, default_bet_bins=BET_BINS,
                        device=torch.device("cpu"), rng=torch.Generator().manual_seed(0))
    decks = []
    for b in boards.tolist():
        unused = [c for c in range(52) if c not in b]
        decks.append(unused[:4] + b + unused[4:5])
    env.reset(force_deck=torch.tensor(decks), force_button=torch.zeros(n, dtype=torch.long))
    for _ in range(4):
        env.step_bins(torch.ones(n, dtype=torch.long))
    assert (env.street == 2).all() and (env.actions_this_round == 0).all()
    env.pot[:] = pot
    env.stacks[:] = stack[:, None]
    env.starting_stacks[:] = (stack + pot // 2)[:, None]
    env.scale[:] = (stack + pot // 2).float()
    if hasattr(env, "raises"):
        env.raises[:] = 0
    return env


def gen_turn() -> None:
    """Turn subgames: every non-fold leaf is the start of the river, valued by the model."""
    import make_golden
    from p2.search.sparse_cfr_evaluator import SparseCFREvaluator

    g = torch.Generator().manual_seed(11)
    n, iterations, cap, depth = 3, 16, 2, 8
    boards = torch.stack([torch.randperm(52, generator=g)[:4] for _ in range(n)])
    ranges = make_golden.dirichlet_ranges(boards, g)
    pot = torch.randint(20, 201, (n,), generator=g)
    stack = torch.randint(100, 1001, (n,), generator=g)
    install_raise_cap(cap)
    ev = make_evaluator(n, iterations, depth=depth)
    ev.model = PotEchoModel(len(BET_BINS) + 3)
    ev.initialize_subgame(turn_env(boards, pot, stack), torch.arange(n), ranges)
    ev.generator = torch.Generator().manual_seed(123)  # consumed by the sampling schedule only
    ev.evaluate_cfr()
    ex = ev._compute_exploitability()
    # leaf sampling (sparse_cfr_evaluator.py:325-426) with a freshly seeded generator
    ev.generator = torch.Generator().manual_seed(321)
    pbs = SparseCFREvaluator.sample_leaves(ev, True)
    ev.generator = torch.Generator().manual_seed(99)
    schedule = ev._get_sampling_schedule()[:n]
    install_raise_cap(None)
    model_mask = ev.leaf_mask & ~ev.env.done
    print("turn nodes", ev.total_nodes, "model leaves", int(model_mask.sum()), "showdown", int((ev.env.street == 4).sum()),
          "exploitability", ex.local_exploitability.tolist())
    save("cfr_turn_cap2_t16.npz",
         boards=boards.to(torch.int16).numpy(), ranges=ranges.numpy(), pot=pot.numpy(), stack=stack.numpy(),
         iterations=np.int64(iterations), cap=np.int64(cap), max_depth=np.int64(depth),
         total_nodes=np.int64(ev.total_nodes), model_mask=model_mask.numpy(), hand_weights=hand_weights().numpy(),
         policy_avg=ev.policy_probs_avg.numpy(), root_values=ev.values_avg[:n].numpy(),
         regrets=ev.cumulative_regrets.numpy(), leaf_mask=ev.leaf_mask.numpy(),
         parent_index=ev.parent_index.numpy(), street=ev.env.street.numpy(),
         t_sample=ev.t_sample[:n].numpy(), policy_sample=ev.policy_probs_sample.numpy(),
         beliefs_last=ev.beliefs.numpy(), sample_epsilon=np.float64(ev.sample_epsilon),
         sampled_beliefs=pbs.beliefs.numpy(), sampled_pot=pbs.env.pot.numpy(),
         sampled_stacks=pbs.env.stacks.numpy(), schedule_seed99=schedule.numpy(),
         exploitability=ex.local_exploitability.numpy(), br_values=ex.local_best_response_values.numpy())


def gen_training_data() -> None:
    """`training_data()` of the upstream evaluator (cfr_evaluator.py:1384-1495) after a short
    river solve: value targets, policy targets, legal masks and statistics."""
    import warnings

    b, r, p, s = seeded_inputs(7, 2, (20, 200), (100, 1000))
    iterations, cap, depth = 12, 2, 8
    install_raise_cap(cap)
    ev = make_evaluator(2, iterations, depth=depth)
    ev.model = PotEchoModel(len(BET_BINS) + 3)  # only the pre-chance batch calls it (no model leaves on the river)
    ev.chance_helper.model = ev.model
    ev.initialize_subgame(river_env(b, p, s), torch.arange(2), r)
    ev.evaluate_cfr()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        vb, pre, pol = ev.training_data(exclude_start=True)
    install_raise_cap(None)
    print("training_data: value", len(vb), "pre", len(pre), "policy", len(pol))
    save("training_data_cap2_t12.npz",
         boards=b.to(torch.int16).numpy(), ranges=r.numpy(), pot=p.numpy(), stack=s.numpy(),
         iterations=np.int64(iterations), cap=np.int64(cap), max_depth=np.int64(depth),
         value_targets=vb.value_targets.numpy(), value_legal_masks=vb.legal_masks.numpy(),
         value_beliefs=vb.features.beliefs.numpy(),
         value_pot=vb.statistics["pot"].numpy(), value_to_act=vb.statistics["to_act"].numpy(),
         value_bet_amounts=vb.statistics["bet_amounts"].numpy(),
         value_exploitability=vb.statistics["local_exploitability"].numpy(),
         value_br=vb.statistics["local_best_response_values"].numpy(),
         policy_targets=pol.policy_targets.numpy(), policy_legal_masks=pol.legal_masks.numpy(),
         policy_beliefs=pol.features.beliefs.numpy(), policy_pot=pol.statistics["pot"].numpy(),
         policy_to_act=pol.statistics["to_act"].numpy(), policy_bet_amounts=pol.statistics["bet_amounts"].numpy(),
         pre_count=np.int64(len(pre)), pre_value_targets=pre.value_targets.numpy(),
         pre_beliefs=pre.features.beliefs.numpy(), pre_board=pre.statistics["board"].numpy(),
         pre_street=pre.statistics["street"].numpy(), pre_stage=pre.statistics["stage"].numpy(),
         hand_weights=hand_weights().numpy())


class FixedLogitModel(ZeroModel):
    """Policy head stand-in: the same logits for every node, a fixed function of (hand, action)."""

    def __call__(self, features, include_policy=True, **kw):
        from p2.models.model_output import ModelOutput

        n = len(features)
        logits = torch.randn(1326, self.num_actions, generator=torch.Generator().manual_seed(31))
        return ModelOutput(policy_logits=logits[None].expand(n, -1, -1).clone(), value=torch.zeros(n),
                           hand_values=torch.zeros(n, 2, 1326))


class BeliefLogitModel(ZeroModel):
    """Policy head stand-in whose logits depend on the node's beliefs: fixed (hand, action) logits plus
    30 x the belief of the player to act in that hand x a per-action weight.  The start policy of a level
    then depends on the beliefs the levels above produced (`initialize_policy_and_beliefs` :832-886)."""

    def __call__(self, features, include_policy=True, **kw):
        from p2.models.model_output import ModelOutput

        n = len(features)
        g = torch.Generator().manual_seed(31)
        fixed = torch.randn(1326, self.num_actions, generator=g)
        w = torch.linspace(-1.0, 1.0, self.num_actions)
        bel = features.beliefs.view(n, 2, 1326).float()
        mine = bel.gather(1, features.to_act.long()[:, None, None].expand(-1, 1, 1326)).squeeze(1)  # [n,1326]
        logits = fixed[None] + 30.0 * mine[:, :, None] * w[None, None, :]
        return ModelOutput(policy_logits=logits, value=torch.zeros(n), hand_values=torch.zeros(n, 2, 1326))


def gen_warm_start() -> None:
    """River subgames with the model's policy as start policy and regrets seeded from it
    (`warm_start`, cfr_evaluator.py:887-926, type `model`), then the remaining iterations."""
    from p2.core.structured_config import WarmStartType

    b, r, p, s = seeded_inputs(13, 2, (20, 200), (100, 1000))
    iterations, ws, mult, cap, depth = 12, 3, 10.0, 2, 8
    install_raise_cap(cap)
    ev = make_evaluator(2, iterations, depth=depth)
    ev.model = FixedLogitModel(len(BET_BINS) + 3)
    ev.warm_start_iterations, ev.warm_start_type, ev.warm_start_multiplier = ws, WarmStartType.model, mult
    captured = {}
    original = ev.warm_start

    def hooked():
        captured["start_policy"] = ev.policy_probs.clone()
        original()
        captured["seeded_regrets"] = ev.cumulative_regrets.clone()
        captured["seeded_weights"] = ev.regret_weight_sums.clone()

    ev.warm_start = hooked
    ev.initialize_subgame(river_env(b, p, s), torch.arange(2), r)
    ev.generator = torch.Generator().manual_seed(5)
    ev.evaluate_cfr()
    ex = ev._compute_exploitability()
    install_raise_cap(None)
    print("warm start nodes", ev.total_nodes, "exploitability", ex.local_exploitability.tolist())
    save("cfr_warm_cap2_t12.npz",
         boards=b.to(torch.int16).numpy(), ranges=r.numpy(), pot=p.numpy(), stack=s.numpy(),
         iterations=np.int64(iterations), warm_start_iterations=np.int64(ws), warm_start_multiplier=np.float64(mult),
         cap=np.int64(cap), max_depth=np.int64(depth), total_nodes=np.int64(ev.total_nodes),
         start_policy=captured["start_policy"].numpy(), seeded_regrets=captured["seeded_regrets"].numpy(),
         seeded_weights=captured["seeded_weights"].numpy(), regrets=ev.cumulative_regrets.numpy(),
         weight_sums=ev.regret_weight_sums.numpy(), policy_avg=ev.policy_probs_avg.numpy(),
         root_values=ev.values_avg[:2].numpy(), t_sample=ev.t_sample[:2].numpy(),
         policy_sample=ev.policy_probs_sample.numpy(), exploitability=ex.local_exploitability.numpy())


SECTIONS = {"tree": gen_tree, "cfr": gen_cfr, "turn": gen_turn, "training_data": gen_training_data,
            "warm_start": gen_warm_start}


class _BeliefEchoModel:
    """Deterministic stand-in for the leaf model of the chance helper: values are a fixed
    function of the sample's beliefs and newest board card."""

    def __init__(self, weights):
        self.w = weights

    def eval(self):
        pass

    def __call__(self, features, **kw):
        from p2.models.model_output import ModelOutput

        n = len(features)
        bel = features.beliefs.view(n, 2, 1326).float()
        newest = features.board.gather(1, ((features.board >= 0).sum(dim=1) - 1).view(-1, 1)).squeeze(1)
        scale = self.w[newest].view(-1, 1, 1)
        hv = torch.stack([bel[:, 1], -bel[:, 0]], dim=1) * scale + 0.25 * scale
        return ModelOutput(policy_logits=None, value=torch.zeros(n), hand_values=hv)


def gen_chance() -> None:
    """single_card_chance_values (chance_node_helper.py:359-479) on turn roots."""
    import warnings

    from p2.models.mlp.mlp_features import MLPFeatures
    from p2.search.chance_node_helper import ChanceNodeHelper

    g = torch.Generator().manual_seed(9)
    B, n_board = 4, 4
    boards = torch.full((B, 5), -1, dtype=torch.long)
    for b in range(B):
        boards[b, :n_board] = torch.randperm(52, generator=g)[:n_board]
    bel = torch.empty(B, 2, 1326).exponential_(generator=g)
    bel = bel / bel.sum(-1, keepdim=True)
    bel[0, 1] = 0
    w = torch.randn(52, generator=torch.Generator().manual_seed(2))
    helper = ChanceNodeHelper(device=torch.device("cpu"), float_dtype=torch.float32, num_players=2,
                              model=_BeliefEchoModel(w), generator=g)
    feats = MLPFeatures(context=torch.zeros(B, 4), street=torch.full((B,), 2), to_act=torch.zeros(B, dtype=torch.long),
                        board=boards, beliefs=bel.reshape(B, -1))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out = helper.single_card_chance_values(torch.arange(B), feats, bel, boards)
    save("chance.npz", boards=boards.numpy(), beliefs=bel.numpy(), weights=w.numpy(), expected=out.numpy())


SECTIONS["chance"] = gen_chance


class _FlopEchoModel:
    """Deterministic stand-in for the leaf model of the flop chance helper: values depend on the
    sample's beliefs, on its three board cards and on the hand index, elementwise."""

    def __init__(self, card_w, hand_w):
        self.cw, self.hw = card_w, hand_w

    def eval(self):
        pass

    def __call__(self, features, **kw):
        from p2.models.model_output import ModelOutput

        n = len(features)
        bel = features.beliefs.view(n, 2, 1326).float()
        scale = self.cw[features.board[:, :3]].sum(dim=1).view(-1, 1, 1)
        hv = torch.stack([bel[:, 1], -bel[:, 0]], dim=1) * scale + self.hw.view(1, 1, -1) * 0.125
        return ModelOutput(policy_logits=None, value=torch.zeros(n), hand_values=hv)


def gen_flop_chance() -> None:
    """flop_chance_values (chance_node_helper.py:218-357): exhaustive over the canonical flops
    with the full suit orbit, and the sampled form (256 flops, 6 permutations)."""
    import warnings

    from p2.models.mlp.mlp_features import MLPFeatures
    from p2.search.chance_node_helper import ChanceNodeHelper

    g = torch.Generator().manual_seed(17)
    B = 2
    bel = torch.empty(B, 2, 1326).exponential_(generator=g)
    bel = bel / bel.sum(-1, keepdim=True)
    cw = torch.randn(52, generator=torch.Generator().manual_seed(3))
    hw = torch.randn(1326, generator=torch.Generator().manual_seed(4))
    helper = ChanceNodeHelper(device=torch.device("cpu"), float_dtype=torch.float32, num_players=2,
                              model=_FlopEchoModel(cw, hw), generator=torch.Generator().manual_seed(23))
    feats = MLPFeatures(context=torch.zeros(B, 4), street=torch.zeros(B), to_act=torch.zeros(B, dtype=torch.long),
                        board=torch.full((B, 5), -1, dtype=torch.long), beliefs=bel.reshape(B, -1))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        sampled = helper.flop_chance_values(torch.arange(B), feats, bel)
        helper.FLOP_SAMPLE_SIZE, helper.NUM_PERM_SAMPLES = 0, 0
        exhaustive = helper.flop_chance_values(torch.arange(B), feats, bel)
    save("flop_chance.npz", beliefs=bel.numpy(), card_w=cw.numpy(), hand_w=hw.numpy(), sampled=sampled.numpy(),
         exhaustive=exhaustive.numpy(), sampled_seed=np.int64(23),
         canonical=helper.flop_id_to_canonical.numpy(), counts=helper.flop_id_to_count.numpy(),
         combo_perm=helper.combo_perm.numpy().astype(np.int16))


SECTIONS["flop_chance"] = gen_flop_chance

"""Two consecutive rounds of the upstream data-generation loop (rebel_data_generator.py:52-95):
initialize_subgame -> evaluate_cfr (with the real leaf sampling) -> training_data, then the same
again from the sampled public states.  Records the environment the first round hands to the second
(every state tensor of the upstream HUNLTensorEnv), the statistics of both rounds and the training
batches of the second.  Imported by make_golden.py."""
from __future__ import annotations

import warnings

import numpy as np
import torch

import golden_cfr as gc
from golden_cfr import BET_BINS, save

ENV_FIELDS = ["button", "street", "to_act", "last_to_act", "pot", "min_raise", "actions_this_round",
              "actions_last_round", "acted_since_reset", "stacks", "committed", "has_folded", "is_allin", "chips_placed",
              "starting_stacks", "scale", "board_indices", "last_board_indices", "hole_indices", "done", "winner",
              "deck", "deck_pos"]


def _env_dump(env, prefix):
    out = {}
    for name in ENV_FIELDS:
        out[f"{prefix}{name}"] = getattr(env, name).numpy()
    if hasattr(env, "raises"):
        out[f"{prefix}raises"] = env.raises.numpy()
    return out


def _stats_dump(stats, prefix):
    out = {}
    for k, v in stats.items():
        if isinstance(v, dict):
            for kk, vv in v.items():
                out[f"{prefix}{k}.{kk}"] = np.float64(vv)
        else:
            out[f"{prefix}{k}"] = np.float64(v)
    return out


def gen_rounds() -> None:
    import make_golden

    g = torch.Generator().manual_seed(41)
    n, iterations, cap, depth = 6, 10, 2, 8
    boards = torch.stack([torch.randperm(52, generator=g)[:4] for _ in range(n)])
    ranges = make_golden.dirichlet_ranges(boards, g)
    pot = torch.randint(20, 201, (n,), generator=g)
    stack = torch.randint(100, 1001, (n,), generator=g)
    gc.install_raise_cap(cap)

    def evaluator(num):
        ev = gc.make_evaluator(num, iterations, depth=depth, enforce_zero_sum=True)
        model = gc.PotEchoModel(len(BET_BINS) + 3)
        model.enforce_zero_sum = True
        ev.model = model
        ev.chance_helper.model = model
        del ev.sample_leaves  # the real sampling walk
        return ev

    ev = evaluator(n)
    env0 = gc.turn_env(boards, pot, stack)
    ev.initialize_subgame(env0, torch.arange(n), ranges)
    ev.generator = torch.Generator().manual_seed(1001)
    pbs = ev.evaluate_cfr()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        vb1, pre1, pol1 = ev.training_data(exclude_start=True)
    n2 = pbs.env.N
    print("round 1: nodes", ev.total_nodes, "continuing states", n2, "streets", pbs.env.street.tolist())
    out = dict(boards=boards.to(torch.int16).numpy(), ranges=ranges.numpy(), pot=pot.numpy(), stack=stack.numpy(),
               iterations=np.int64(iterations), cap=np.int64(cap), max_depth=np.int64(depth),
               hand_weights=gc.hand_weights().numpy(), seed_round1=np.int64(1001), seed_round2=np.int64(1002),
               sample_epsilon=np.float64(ev.sample_epsilon))
    out.update(_env_dump(env0, "env0_"))
    out.update(_env_dump(pbs.env, "env1_"))
    out["beliefs1"] = pbs.beliefs.numpy()
    out.update(_stats_dump(ev.stats, "stats1_"))
    out["value_targets1"] = vb1.value_targets.numpy()

    ev2 = evaluator(n2)
    ev2.initialize_subgame(pbs.env, torch.arange(n2), pbs.beliefs)
    ev2.generator = torch.Generator().manual_seed(1002)
    pbs2 = ev2.evaluate_cfr()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        vb2, pre2, pol2 = ev2.training_data(exclude_start=True)
    gc.install_raise_cap(None)
    print("round 2: nodes", ev2.total_nodes, "value", len(vb2), "pre", len(pre2), "policy", len(pol2),
          "continuing", pbs2.env.N)
    out.update(_stats_dump(ev2.stats, "stats2_"))
    rows = np.arange(0, len(pol2), 5, dtype=np.int64)
    out.update(
        total_nodes2=np.int64(ev2.total_nodes),
        value_targets2=vb2.value_targets.numpy(), value_beliefs2=vb2.features.beliefs.numpy(),
        value_board2=vb2.features.board.numpy(), value_context2=vb2.features.context.numpy(),
        value_street2=vb2.features.street.numpy(), value_to_act2=vb2.features.to_act.numpy(),
        value_legal2=vb2.legal_masks.numpy(), value_pot2=vb2.statistics["pot"].numpy(),
        value_exploitability2=vb2.statistics["local_exploitability"].numpy(),
        pre_value_targets2=pre2.value_targets.numpy(), pre_beliefs2=pre2.features.beliefs.numpy(),
        pre_board2=pre2.features.board.numpy(), pre_street2=pre2.statistics["street"].numpy(),
        policy_rows2=rows, policy_targets2=pol2.policy_targets[torch.from_numpy(rows)].numpy(),
        policy_beliefs2=pol2.features.beliefs[torch.from_numpy(rows)].numpy(), policy_count2=np.int64(len(pol2)),
        continuing2=np.int64(pbs2.env.N))
    save("rounds_turn_river.npz", **out)


gc.SECTIONS.update(rounds=gen_rounds)

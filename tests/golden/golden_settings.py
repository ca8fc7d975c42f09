"""Golden vectors for solver settings beyond plain DCFR (runs the upstream evaluator): the
search block of the upstream production configuration, standard CFR, zero-sum enforcement of
the value targets, and the headline workload at depth (ragged roots x 256 iterations).

Imported by make_golden.py; same river / turn set-up as golden_cfr.py.
"""
from __future__ import annotations

import numpy as np
import torch

import golden_cfr as gc
from golden_cfr import BET_BINS, save


def _solve(ev, env, n, ranges, seed=5):
    ev.initialize_subgame(env, torch.arange(n), ranges)
    ev.generator = torch.Generator().manual_seed(seed)  # consumed by the sampling schedule only
    ev.evaluate_cfr()
    return ev._compute_exploitability()


def gen_production() -> None:
    """The search block of conf/config_rebel_cfr.yaml:78-94 (discounted_plus with a delay, exponent
    schedules alpha 2->4, beta -1->-2, gamma 5->0, warm start of type `model` with 15 iterations and
    multiplier 10) at a reduced iteration count, with a zero-sum model like the production default."""
    from p2.core.structured_config import CFRType, WarmStartType

    b, r, p, s = gc.seeded_inputs(21, 2, (20, 200), (100, 1000))
    iterations, ws, delay, cap, depth = 40, 15, 24, 2, 8
    search = dict(cfr_type=CFRType.discounted_plus, dcfr_plus_delay=delay, warm_start_iterations=ws,
                  warm_start_type=WarmStartType.model, warm_start_multiplier=10.0,
                  dcfr_alpha=2.0, dcfr_alpha_final=4.0, dcfr_beta=-1.0, dcfr_beta_final=-2.0,
                  dcfr_gamma=5.0, dcfr_gamma_final=0.0)
    gc.install_raise_cap(cap)
    ev = gc.make_evaluator(2, iterations, depth=depth, search=search, enforce_zero_sum=True)
    model = gc.FixedLogitModel(len(BET_BINS) + 3)
    model.enforce_zero_sum = True
    ev.model = model
    captured = {}
    original = ev.warm_start

    def hooked():
        captured["start_policy"] = ev.policy_probs.clone()
        original()

    ev.warm_start = hooked
    ex = _solve(ev, gc.river_env(b, p, s), 2, r)
    gc.install_raise_cap(None)
    print("production block: nodes", ev.total_nodes, "exploitability", ex.local_exploitability.tolist())
    save("cfr_production_cap2_t40.npz",
         boards=b.to(torch.int16).numpy(), ranges=r.numpy(), pot=p.numpy(), stack=s.numpy(),
         iterations=np.int64(iterations), warm_start_iterations=np.int64(ws), warm_start_multiplier=np.float64(10.0),
         dcfr_delay=np.int64(delay), cap=np.int64(cap), max_depth=np.int64(depth),
         alpha=np.float64([2.0, 4.0]), beta=np.float64([-1.0, -2.0]), gamma=np.float64([5.0, 0.0]),
         total_nodes=np.int64(ev.total_nodes), start_policy=captured["start_policy"].numpy(),
         regrets=ev.cumulative_regrets.numpy(), weight_sums=ev.regret_weight_sums.numpy(),
         policy_avg=ev.policy_probs_avg.numpy(), root_values=ev.values_avg[:2].numpy(),
         values_avg=ev.values_avg.numpy(), t_sample=ev.t_sample[:2].numpy(),
         policy_sample=ev.policy_probs_sample.numpy(), exploitability=ex.local_exploitability.numpy())


def gen_standard() -> None:
    """cfr_type = standard (no discounting, mixing weights (t, 1)), 16 iterations."""
    from p2.core.structured_config import CFRType

    b, r, p, s = gc.seeded_inputs(22, 2, (20, 200), (100, 1000))
    iterations, cap, depth = 16, 2, 8
    gc.install_raise_cap(cap)
    ev = gc.make_evaluator(2, iterations, depth=depth, search=dict(cfr_type=CFRType.standard))
    ex = _solve(ev, gc.river_env(b, p, s), 2, r)
    gc.install_raise_cap(None)
    print("standard CFR: nodes", ev.total_nodes, "exploitability", ex.local_exploitability.tolist())
    save("cfr_standard_cap2_t16.npz",
         boards=b.to(torch.int16).numpy(), ranges=r.numpy(), pot=p.numpy(), stack=s.numpy(),
         iterations=np.int64(iterations), cap=np.int64(cap), max_depth=np.int64(depth),
         total_nodes=np.int64(ev.total_nodes), regrets=ev.cumulative_regrets.numpy(),
         weight_sums=ev.regret_weight_sums.numpy(), policy_avg=ev.policy_probs_avg.numpy(),
         root_values=ev.values_avg[:2].numpy(), exploitability=ex.local_exploitability.numpy())


def gen_zero_sum() -> None:
    """Value targets with `model.enforce_zero_sum = True` (the model-config default): the shift of
    `update_average_values_final` (cfr_evaluator.py:1289-1292) on river subgames, and on turn
    subgames whose model leaves are shifted too."""
    b, r, p, s = gc.seeded_inputs(23, 2, (20, 200), (100, 1000))
    iterations, cap, depth = 12, 2, 8
    gc.install_raise_cap(cap)
    ev = gc.make_evaluator(2, iterations, depth=depth, enforce_zero_sum=True)
    ex = _solve(ev, gc.river_env(b, p, s), 2, r)
    river = dict(
        river_boards=b.to(torch.int16).numpy(), river_ranges=r.numpy(), river_pot=p.numpy(), river_stack=s.numpy(),
        river_iterations=np.int64(iterations), river_total_nodes=np.int64(ev.total_nodes),
        river_policy_avg=ev.policy_probs_avg.numpy(), river_values_avg=ev.values_avg.numpy(),
        river_beliefs_avg=ev.beliefs_avg.numpy(), river_exploitability=ex.local_exploitability.numpy())
    print("zero-sum river: nodes", ev.total_nodes, "exploitability", ex.local_exploitability.tolist())

    g = torch.Generator().manual_seed(24)
    n, iterations_t = 3, 10
    import make_golden
    boards = torch.stack([torch.randperm(52, generator=g)[:4] for _ in range(n)])
    ranges = make_golden.dirichlet_ranges(boards, g)
    pot = torch.randint(20, 201, (n,), generator=g)
    stack = torch.randint(100, 1001, (n,), generator=g)
    ev = gc.make_evaluator(n, iterations_t, depth=depth, enforce_zero_sum=True)
    model = gc.PotEchoModel(len(BET_BINS) + 3)
    model.enforce_zero_sum = True
    ev.model = model
    ex = _solve(ev, gc.turn_env(boards, pot, stack), n, ranges, seed=123)
    gc.install_raise_cap(None)
    model_mask = ev.leaf_mask & ~ev.env.done
    print("zero-sum turn: nodes", ev.total_nodes, "model leaves", int(model_mask.sum()),
          "exploitability", ex.local_exploitability.tolist())
    save("cfr_zero_sum.npz", cap=np.int64(cap), max_depth=np.int64(depth), **river,
         turn_boards=boards.to(torch.int16).numpy(), turn_ranges=ranges.numpy(), turn_pot=pot.numpy(),
         turn_stack=stack.numpy(), turn_iterations=np.int64(iterations_t), turn_total_nodes=np.int64(ev.total_nodes),
         turn_model_mask=model_mask.numpy(), hand_weights=gc.hand_weights().numpy(),
         turn_policy_avg=ev.policy_probs_avg.numpy(), turn_values_avg=ev.values_avg.numpy(),
         turn_exploitability=ex.local_exploitability.numpy(), turn_br_values=ex.local_best_response_values.numpy())


def gen_ragged256() -> None:
    """The headline workload at depth: 16 ragged river roots (pot U[20,200], stack U[100,1000]),
    max 2 raises, DCFR(1.5, 0, 2), 256 iterations.  Kept small: root values, exploitability and a
    fixed subsample of the average-policy rows."""
    n, iterations, cap, depth = 16, 256, 2, 8
    b, r, p, s = gc.seeded_inputs(2, n, (20, 200), (100, 1000))
    gc.install_raise_cap(cap)
    ev = gc.make_evaluator(n, iterations, depth=depth)
    ex = _solve(ev, gc.river_env(b, p, s), n, r)
    gc.install_raise_cap(None)
    rows = np.arange(n, ev.total_nodes, 11, dtype=np.int64)  # every 11th non-root node, upstream order
    print("ragged x256: nodes", ev.total_nodes, "rows kept", len(rows), "exploitability",
          ex.local_exploitability.tolist()[:4])
    save("cfr_ragged16_cap2_t256.npz",
         boards=b.to(torch.int16).numpy(), ranges=r.numpy(), pot=p.numpy(), stack=s.numpy(),
         iterations=np.int64(iterations), cap=np.int64(cap), max_depth=np.int64(depth),
         total_nodes=np.int64(ev.total_nodes), policy_rows=rows,
         policy_avg_rows=ev.policy_probs_avg[torch.from_numpy(rows)].numpy(),
         regret_rows=ev.cumulative_regrets[torch.from_numpy(rows)].numpy(),
         root_values=ev.values_avg[:n].numpy(), exploitability=ex.local_exploitability.numpy(),
         br_values=ex.local_best_response_values.numpy())


def gen_cfr_avg() -> None:
    """`cfr_avg = True` (the dataclass default upstream; cfr_evaluator.py:997-1018, :1029, :1133): leaf
    values and regret weights from the beliefs under the average policy, and the model's leaf values
    de-averaged from the second iteration on.  River subgames (showdown leaves at the average beliefs)
    and turn subgames with a stand-in model, both with the zero-sum shift on."""
    b, r, p, s = gc.seeded_inputs(31, 2, (20, 200), (100, 1000))
    iterations, cap, depth = 12, 2, 8
    gc.install_raise_cap(cap)
    ev = gc.make_evaluator(2, iterations, depth=depth, search=dict(cfr_avg=True), enforce_zero_sum=True)
    ex = _solve(ev, gc.river_env(b, p, s), 2, r)
    river = dict(
        river_boards=b.to(torch.int16).numpy(), river_ranges=r.numpy(), river_pot=p.numpy(), river_stack=s.numpy(),
        river_iterations=np.int64(iterations), river_total_nodes=np.int64(ev.total_nodes),
        river_policy_avg=ev.policy_probs_avg.numpy(), river_regrets=ev.cumulative_regrets.numpy(),
        river_values_avg=ev.values_avg.numpy(), river_exploitability=ex.local_exploitability.numpy())
    print("cfr_avg river: nodes", ev.total_nodes, "exploitability", ex.local_exploitability.tolist())

    g = torch.Generator().manual_seed(32)
    n, iterations_t = 2, 10
    import make_golden
    boards = torch.stack([torch.randperm(52, generator=g)[:4] for _ in range(n)])
    ranges = make_golden.dirichlet_ranges(boards, g)
    pot = torch.randint(20, 201, (n,), generator=g)
    stack = torch.randint(100, 1001, (n,), generator=g)
    ev = gc.make_evaluator(n, iterations_t, depth=depth, search=dict(cfr_avg=True), enforce_zero_sum=True)
    model = gc.PotEchoModel(len(BET_BINS) + 3)
    model.enforce_zero_sum = True
    ev.model = model
    ex = _solve(ev, gc.turn_env(boards, pot, stack), n, ranges, seed=123)
    gc.install_raise_cap(None)
    model_mask = ev.leaf_mask & ~ev.env.done
    print("cfr_avg turn: nodes", ev.total_nodes, "model leaves", int(model_mask.sum()),
          "exploitability", ex.local_exploitability.tolist())
    save("cfr_avg.npz", cap=np.int64(cap), max_depth=np.int64(depth), **river,
         turn_boards=boards.to(torch.int16).numpy(), turn_ranges=ranges.numpy(), turn_pot=pot.numpy(),
         turn_stack=stack.numpy(), turn_iterations=np.int64(iterations_t), turn_total_nodes=np.int64(ev.total_nodes),
         turn_model_mask=model_mask.numpy(), hand_weights=gc.hand_weights().numpy(),
         turn_policy_avg=ev.policy_probs_avg.numpy(), turn_regrets=ev.cumulative_regrets.numpy(),
         turn_values_avg=ev.values_avg.numpy(), turn_exploitability=ex.local_exploitability.numpy(),
         turn_br_values=ex.local_best_response_values.numpy())


def gen_running_values() -> None:
    """`value_targets_from_final_policy = False` (the dataclass default upstream): values_avg is the running
    mix of the per-iteration values with the zero-sum shift applied every iteration
    (`update_average_values`, cfr_evaluator.py:1260-1274); no final pass.  River and turn subgames."""
    b, r, p, s = gc.seeded_inputs(41, 2, (20, 200), (100, 1000))
    iterations, cap, depth = 12, 2, 8
    gc.install_raise_cap(cap)
    search = dict(value_targets_from_final_policy=False)
    ev = gc.make_evaluator(2, iterations, depth=depth, search=search, enforce_zero_sum=True)
    ex = _solve(ev, gc.river_env(b, p, s), 2, r)
    river = dict(
        river_boards=b.to(torch.int16).numpy(), river_ranges=r.numpy(), river_pot=p.numpy(), river_stack=s.numpy(),
        river_iterations=np.int64(iterations), river_total_nodes=np.int64(ev.total_nodes),
        river_policy_avg=ev.policy_probs_avg.numpy(), river_values_avg=ev.values_avg.numpy(),
        river_exploitability=ex.local_exploitability.numpy(), river_br_values=ex.local_best_response_values.numpy())
    print("running values river: nodes", ev.total_nodes, "exploitability", ex.local_exploitability.tolist())

    g = torch.Generator().manual_seed(42)
    n, iterations_t = 2, 10
    import make_golden
    boards = torch.stack([torch.randperm(52, generator=g)[:4] for _ in range(n)])
    ranges = make_golden.dirichlet_ranges(boards, g)
    pot = torch.randint(20, 201, (n,), generator=g)
    stack = torch.randint(100, 1001, (n,), generator=g)
    ev = gc.make_evaluator(n, iterations_t, depth=depth, search=search, enforce_zero_sum=True)
    model = gc.PotEchoModel(len(BET_BINS) + 3)
    model.enforce_zero_sum = True
    ev.model = model
    ex = _solve(ev, gc.turn_env(boards, pot, stack), n, ranges, seed=123)
    gc.install_raise_cap(None)
    model_mask = ev.leaf_mask & ~ev.env.done
    print("running values turn: nodes", ev.total_nodes, "model leaves", int(model_mask.sum()),
          "exploitability", ex.local_exploitability.tolist())
    save("cfr_running_values.npz", cap=np.int64(cap), max_depth=np.int64(depth), **river,
         turn_boards=boards.to(torch.int16).numpy(), turn_ranges=ranges.numpy(), turn_pot=pot.numpy(),
         turn_stack=stack.numpy(), turn_iterations=np.int64(iterations_t), turn_total_nodes=np.int64(ev.total_nodes),
         turn_model_mask=model_mask.numpy(), hand_weights=gc.hand_weights().numpy(),
         turn_policy_avg=ev.policy_probs_avg.numpy(), turn_values_avg=ev.values_avg.numpy(),
         turn_exploitability=ex.local_exploitability.numpy(), turn_br_values=ex.local_best_response_values.numpy())


def gen_warm_br() -> None:
    """Warm start of type `model_br` (the dataclass default upstream; cfr_evaluator.py:927-955): regrets seeded
    with the regrets of not playing a best response against the model's policy.  River subgames with a fixed
    policy head, and turn subgames with a stand-in value model."""
    from p2.core.structured_config import WarmStartType

    out = {}
    for tag, seed in (("river", 51), ("turn", 52)):
        iterations, ws, mult, cap, depth = 10, 3, 4.0, 2, 8
        gc.install_raise_cap(cap)
        ev = gc.make_evaluator(2, iterations, depth=depth)
        if tag == "river":
            b, r, p, s = gc.seeded_inputs(seed, 2, (20, 200), (100, 1000))
            ev.model = gc.FixedLogitModel(len(BET_BINS) + 3)
            env = gc.river_env(b, p, s)
        else:
            g = torch.Generator().manual_seed(seed)
            import make_golden
            b = torch.stack([torch.randperm(52, generator=g)[:4] for _ in range(2)])
            r = make_golden.dirichlet_ranges(b, g)
            p = torch.randint(20, 201, (2,), generator=g)
            s = torch.randint(100, 1001, (2,), generator=g)

            class Both(gc.PotEchoModel):  # value head of PotEchoModel, policy head of FixedLogitModel
                def __call__(self, features, include_policy=True, **kw):
                    o = gc.PotEchoModel.__call__(self, features, include_policy, **kw)
                    o.policy_logits = gc.FixedLogitModel.__call__(self, features, include_policy, **kw).policy_logits
                    return o

            ev.model = Both(len(BET_BINS) + 3)
            env = gc.turn_env(b, p, s)
        ev.warm_start_iterations, ev.warm_start_type, ev.warm_start_multiplier = ws, WarmStartType.model_br, mult
        captured = {}
        original = ev.warm_start

        def hooked(ev=ev, captured=captured, original=original):
            captured["start_policy"] = ev.policy_probs.clone()
            original()
            captured["seeded_regrets"] = ev.cumulative_regrets.clone()

        ev.warm_start = hooked
        ex = _solve(ev, env, 2, r)
        gc.install_raise_cap(None)
        model_mask = ev.leaf_mask & ~ev.env.done
        print(f"model_br warm start, {tag}: nodes", ev.total_nodes, "exploitability", ex.local_exploitability.tolist())
        out.update({f"{tag}_boards": b.to(torch.int16).numpy(), f"{tag}_ranges": r.numpy(), f"{tag}_pot": p.numpy(),
                    f"{tag}_stack": s.numpy(), f"{tag}_total_nodes": np.int64(ev.total_nodes),
                    f"{tag}_model_mask": model_mask.numpy(), f"{tag}_start_policy": captured["start_policy"].numpy(),
                    f"{tag}_seeded_regrets": captured["seeded_regrets"].numpy(),
                    f"{tag}_policy_avg": ev.policy_probs_avg.numpy(),
                    f"{tag}_root_values": ev.values_avg[:2].numpy(),
                    f"{tag}_exploitability": ex.local_exploitability.numpy()})
    save("cfr_warm_br.npz", iterations=np.int64(10), warm_start_iterations=np.int64(3),
         warm_start_multiplier=np.float64(4.0), cap=np.int64(2), max_depth=np.int64(8),
         hand_weights=gc.hand_weights().numpy(), **out)


def gen_linear() -> None:
    """cfr_type = linear (the dataclass default upstream): no discounting, alternating updates (the actions of
    player t % 2 get no regret at iteration t, cfr_evaluator.py:1348-1349), mixing weights (t, 2); with the CFR+
    clamp the dataclass default also sets.  River subgames, 13 iterations."""
    from p2.core.structured_config import CFRType

    b, r, p, s = gc.seeded_inputs(61, 2, (20, 200), (100, 1000))
    iterations, cap, depth = 13, 2, 8
    gc.install_raise_cap(cap)
    ev = gc.make_evaluator(2, iterations, depth=depth, search=dict(cfr_type=CFRType.linear, cfr_plus=True))
    ex = _solve(ev, gc.river_env(b, p, s), 2, r)
    gc.install_raise_cap(None)
    print("linear CFR: nodes", ev.total_nodes, "exploitability", ex.local_exploitability.tolist())
    save("cfr_linear_cap2_t13.npz",
         boards=b.to(torch.int16).numpy(), ranges=r.numpy(), pot=p.numpy(), stack=s.numpy(),
         iterations=np.int64(iterations), cap=np.int64(cap), max_depth=np.int64(depth),
         total_nodes=np.int64(ev.total_nodes), regrets=ev.cumulative_regrets.numpy(),
         weight_sums=ev.regret_weight_sums.numpy(), policy_avg=ev.policy_probs_avg.numpy(),
         root_values=ev.values_avg[:2].numpy(), exploitability=ex.local_exploitability.numpy())


def gen_policy_head() -> None:
    """Start policy from a policy head that reads the node beliefs, level by level
    (`initialize_policy_and_beliefs`, cfr_evaluator.py:832-886), then a warm start of type `model` and the
    remaining iterations.  River subgames."""
    from p2.core.structured_config import WarmStartType

    b, r, p, s = gc.seeded_inputs(71, 2, (20, 200), (100, 1000))
    iterations, ws, mult, cap, depth = 8, 2, 5.0, 2, 8
    gc.install_raise_cap(cap)
    ev = gc.make_evaluator(2, iterations, depth=depth)
    ev.model = gc.BeliefLogitModel(len(BET_BINS) + 3)
    ev.warm_start_iterations, ev.warm_start_type, ev.warm_start_multiplier = ws, WarmStartType.model, mult
    captured = {}
    original = ev.warm_start

    def hooked():
        captured["start_policy"] = ev.policy_probs.clone()
        captured["start_beliefs"] = ev.beliefs.clone()
        original()

    ev.warm_start = hooked
    ex = _solve(ev, gc.river_env(b, p, s), 2, r)
    gc.install_raise_cap(None)
    print("policy head: nodes", ev.total_nodes, "exploitability", ex.local_exploitability.tolist())
    save("cfr_policy_head.npz",
         boards=b.to(torch.int16).numpy(), ranges=r.numpy(), pot=p.numpy(), stack=s.numpy(),
         iterations=np.int64(iterations), warm_start_iterations=np.int64(ws), warm_start_multiplier=np.float64(mult),
         cap=np.int64(cap), max_depth=np.int64(depth), total_nodes=np.int64(ev.total_nodes),
         start_policy=captured["start_policy"].numpy(), start_beliefs=captured["start_beliefs"].numpy(),
         policy_avg=ev.policy_probs_avg.numpy(), root_values=ev.values_avg[:2].numpy(),
         exploitability=ex.local_exploitability.numpy())


def gen_dataclass_defaults() -> None:
    """The search settings a bare `SearchConfig()` gives (structured_config.py:236-265), all at once: linear CFR
    with the CFR+ clamp, `cfr_avg`, value targets from the running average, warm start of type `model_br`
    (3 of 9 iterations here), zero-sum model.  River subgames with a fixed policy head, turn subgames with a
    stand-in value model."""
    from p2.core.structured_config import CFRType, WarmStartType

    out = {}
    for tag, seed in (("river", 81), ("turn", 82)):
        iterations, ws, mult, cap, depth = 9, 3, 1.0, 2, 8
        gc.install_raise_cap(cap)
        search = dict(cfr_type=CFRType.linear, cfr_plus=True, cfr_avg=True, value_targets_from_final_policy=False)
        ev = gc.make_evaluator(2, iterations, depth=depth, search=search, enforce_zero_sum=True)
        if tag == "river":
            b, r, p, s = gc.seeded_inputs(seed, 2, (20, 200), (100, 1000))
            model = gc.FixedLogitModel(len(BET_BINS) + 3)
            env = gc.river_env(b, p, s)
        else:
            g = torch.Generator().manual_seed(seed)
            import make_golden
            b = torch.stack([torch.randperm(52, generator=g)[:4] for _ in range(2)])
            r = make_golden.dirichlet_ranges(b, g)
            p = torch.randint(20, 201, (2,), generator=g)
            s = torch.randint(100, 1001, (2,), generator=g)

            class Both(gc.PotEchoModel):
                def __call__(self, features, include_policy=True, **kw):
                    o = gc.PotEchoModel.__call__(self, features, include_policy, **kw)
                    o.policy_logits = gc.FixedLogitModel.__call__(self, features, include_policy, **kw).policy_logits
                    return o

            model = Both(len(BET_BINS) + 3)
            env = gc.turn_env(b, p, s)
        model.enforce_zero_sum = True
        ev.model = model
        ev.warm_start_iterations, ev.warm_start_type, ev.warm_start_multiplier = ws, WarmStartType.model_br, mult
        captured = {}
        original = ev.warm_start

        def hooked(ev=ev, captured=captured, original=original):
            captured["start_policy"] = ev.policy_probs.clone()
            original()

        ev.warm_start = hooked
        ex = _solve(ev, env, 2, r)
        gc.install_raise_cap(None)
        model_mask = ev.leaf_mask & ~ev.env.done
        print(f"dataclass defaults, {tag}: nodes", ev.total_nodes, "exploitability", ex.local_exploitability.tolist())
        out.update({f"{tag}_boards": b.to(torch.int16).numpy(), f"{tag}_ranges": r.numpy(), f"{tag}_pot": p.numpy(),
                    f"{tag}_stack": s.numpy(), f"{tag}_total_nodes": np.int64(ev.total_nodes),
                    f"{tag}_model_mask": model_mask.numpy(), f"{tag}_start_policy": captured["start_policy"].numpy(),
                    f"{tag}_policy_avg": ev.policy_probs_avg.numpy(), f"{tag}_regrets": ev.cumulative_regrets.numpy(),
                    f"{tag}_root_values": ev.values_avg[:2].numpy(),
                    f"{tag}_exploitability": ex.local_exploitability.numpy()})
    save("cfr_dataclass_defaults.npz", iterations=np.int64(9), warm_start_iterations=np.int64(3),
         warm_start_multiplier=np.float64(1.0), cap=np.int64(2), max_depth=np.int64(8),
         hand_weights=gc.hand_weights().numpy(), **out)


def gen_policy_delta() -> None:
    """The `cfr_delta.*` statistics (`_record_stats`, cfr_evaluator.py:1573-1605): mean absolute change of the
    policy over the reachable hands at the iterations linspace(warm start, T - 1, 5).  Three river solves:
    plain DCFR; three iterations only (the five points collide, the first key of a collision is the one
    written); a warm start of type `model` from a policy head."""
    from p2.core.structured_config import WarmStartType

    out = {}
    cap, depth = 2, 8
    for tag, seed, iterations, ws in (("plain", 81, 9, 0), ("short", 82, 3, 0), ("warm", 83, 10, 3)):
        b, r, p, s = gc.seeded_inputs(seed, 2, (20, 200), (100, 1000))
        gc.install_raise_cap(cap)
        ev = gc.make_evaluator(2, iterations, depth=depth)
        captured = {}
        if ws:
            ev.model = gc.BeliefLogitModel(len(BET_BINS) + 3)
            ev.warm_start_iterations, ev.warm_start_type, ev.warm_start_multiplier = ws, WarmStartType.model, 4.0
            original = ev.warm_start

            def hooked(ev=ev, captured=captured, original=original):
                captured["start_policy"] = ev.policy_probs.clone()
                original()

            ev.warm_start = hooked
        ex = _solve(ev, gc.river_env(b, p, s), 2, r)
        gc.install_raise_cap(None)
        deltas = {k: v for k, v in ev.stats.items() if k.startswith("cfr_delta.")}
        print(f"policy delta, {tag}: nodes", ev.total_nodes, deltas)
        out.update({f"{tag}_boards": b.to(torch.int16).numpy(), f"{tag}_ranges": r.numpy(), f"{tag}_pot": p.numpy(),
                    f"{tag}_stack": s.numpy(), f"{tag}_iterations": np.int64(iterations),
                    f"{tag}_warm_start_iterations": np.int64(ws), f"{tag}_total_nodes": np.int64(ev.total_nodes),
                    f"{tag}_exploitability": ex.local_exploitability.numpy(),
                    f"{tag}_delta_keys": np.array(sorted(int(k.split(".")[1]) for k in deltas), dtype=np.int64),
                    f"{tag}_delta_values": np.array([deltas[f"cfr_delta.{q}"] for q in
                                                     sorted(int(k.split(".")[1]) for k in deltas)], dtype=np.float64)})
        if ws:
            out[f"{tag}_start_policy"] = captured["start_policy"].numpy()
    save("cfr_policy_delta.npz", cap=np.int64(cap), max_depth=np.int64(depth), warm_start_multiplier=np.float64(4.0),
         **out)


def gen_depth5() -> None:
    """The tree shape of the production search settings (conf/config_rebel_cfr.yaml:65-73: bet sizes {0.5, 1.0},
    depth 5, no raise cap) on turn roots with deep stacks: 273 nodes per root, 68 of them internal, leaves at
    depth 5 and at the start of the river valued by the stand-in model.  Stores root values, exploitability and
    every 7th row of the average policy and the regrets."""
    import make_golden

    g = torch.Generator().manual_seed(91)
    n, iterations, depth = 2, 6, 5
    boards = torch.stack([torch.randperm(52, generator=g)[:4] for _ in range(n)])
    ranges = make_golden.dirichlet_ranges(boards, g)
    pot, stack = torch.tensor([20, 60]), torch.tensor([990, 970])
    gc.install_raise_cap(None)
    ev = gc.make_evaluator(n, iterations, depth=depth)
    ev.model = gc.PotEchoModel(len(BET_BINS) + 3)
    ev.initialize_subgame(gc.turn_env(boards, pot, stack), torch.arange(n), ranges)
    ev.generator = torch.Generator().manual_seed(5)
    ev.evaluate_cfr()
    ex = ev._compute_exploitability()
    model_mask = ev.leaf_mask & ~ev.env.done
    rows = torch.arange(n, ev.total_nodes, 7)
    print("depth 5, no cap: nodes", ev.total_nodes, "model leaves", int(model_mask.sum()), "exploitability",
          ex.local_exploitability.tolist())
    save("cfr_depth5_nocap_t6.npz",
         boards=boards.to(torch.int16).numpy(), ranges=ranges.numpy(), pot=pot.numpy(), stack=stack.numpy(),
         iterations=np.int64(iterations), max_depth=np.int64(depth), total_nodes=np.int64(ev.total_nodes),
         model_mask=model_mask.numpy(), hand_weights=gc.hand_weights().numpy(), rows=rows.numpy(),
         policy_avg_rows=ev.policy_probs_avg[rows].numpy(), regrets_rows=ev.cumulative_regrets[rows].numpy(),
         root_values=ev.values_avg[:n].numpy(), exploitability=ex.local_exploitability.numpy(),
         br_values=ex.local_best_response_values.numpy())


def gen_default_bins() -> None:
    """The bet sizes of the upstream configuration dataclass ({0.5, 0.75, 1.0, 1.5, 2.0}: eight actions per
    node) on river roots at depth 3 without a raise cap: trees of up to 280 nodes whose deepest leaves are
    valued by the stand-in model.  Stores root values, exploitability and every 5th row of the average policy
    and the regrets."""
    bins = [0.5, 0.75, 1.0, 1.5, 2.0]
    b, r, p, s = gc.seeded_inputs(93, 2, (20, 200), (100, 1000))
    p, s = torch.tensor([40, 100]), torch.tensor([1000, 400])
    iterations, depth = 6, 3
    old = gc.BET_BINS
    gc.BET_BINS = bins
    try:
        gc.install_raise_cap(None)
        ev = gc.make_evaluator(2, iterations, depth=depth)
        ev.model = gc.PotEchoModel(len(bins) + 3)
        ex = _solve(ev, gc.river_env(b, p, s), 2, r)
    finally:
        gc.BET_BINS = old
    model_mask = ev.leaf_mask & ~ev.env.done
    rows = torch.arange(2, ev.total_nodes, 5)
    print("default bet sizes: nodes", ev.total_nodes, "actions", ev.num_actions, "model leaves", int(model_mask.sum()),
          "exploitability", ex.local_exploitability.tolist())
    save("cfr_default_bins_depth3_t6.npz",
         boards=b.to(torch.int16).numpy(), ranges=r.numpy(), pot=p.numpy(), stack=s.numpy(), bet_bins=np.float64(bins),
         iterations=np.int64(iterations), max_depth=np.int64(depth), total_nodes=np.int64(ev.total_nodes),
         model_mask=model_mask.numpy(), hand_weights=gc.hand_weights().numpy(), rows=rows.numpy(),
         policy_avg_rows=ev.policy_probs_avg[rows].numpy(), regrets_rows=ev.cumulative_regrets[rows].numpy(),
         root_values=ev.values_avg[:2].numpy(), exploitability=ex.local_exploitability.numpy(),
         br_values=ex.local_best_response_values.numpy())


gc.SECTIONS.update(production=gen_production, standard=gen_standard, zero_sum=gen_zero_sum, ragged256=gen_ragged256,
                   cfr_avg=gen_cfr_avg, running_values=gen_running_values, warm_br=gen_warm_br, linear=gen_linear, policy_head=gen_policy_head, dataclass_defaults=gen_dataclass_defaults,
                   policy_delta=gen_policy_delta, depth5=gen_depth5,
                   default_bins=gen_default_bins)

"""The CFR oracle under solver settings beyond plain DCFR, against arrays produced by the upstream
evaluator: the production search block (discounted_plus, delay, exponent schedules, warm start),
standard CFR, zero-sum value targets, and iteration_scalars against the oracle's own schedule."""
import os

import numpy as np
import pytest
import torch

from leaf_models import pot_echo_leaf_fn
from oracle import cfr as ocfr
from poker2_b200 import solver, tree as ptree

BET_BINS = [0.5, 1.0]


def _build(pot, stack, cap, depth, street=3):
    roots = ptree.root_states(pot, stack, min_raise=2, street=street)
    return ptree.build_trees(roots, BET_BINS, depth, bb=2, max_raises=cap)


def test_oracle_production_search_block_bit_exact(golden_dir):
    z = np.load(os.path.join(golden_dir, "cfr_production_cap2_t40.npz"))
    t = _build(z["pot"], z["stack"], int(z["cap"]), int(z["max_depth"]))
    assert t.total_nodes == int(z["total_nodes"])
    o = ocfr.SubgameOracle(
        t.oracle_dict(z["boards"].astype(np.int64)), torch.from_numpy(z["ranges"]), iterations=int(z["iterations"]),
        cfr_type="discounted_plus", dcfr_delay=int(z["dcfr_delay"]), alpha=float(z["alpha"][0]),
        alpha_final=float(z["alpha"][1]), beta=float(z["beta"][0]), beta_final=float(z["beta"][1]),
        gamma=float(z["gamma"][0]), gamma_final=float(z["gamma"][1]), start_policy=torch.from_numpy(z["start_policy"]),
        warm_start_iterations=int(z["warm_start_iterations"]), warm_start_multiplier=float(z["warm_start_multiplier"]),
        enforce_zero_sum=True).solve()
    assert torch.equal(o.regrets, torch.from_numpy(z["regrets"]))
    assert torch.equal(o.weight_sums, torch.from_numpy(z["weight_sums"]))
    assert torch.equal(o.policy_avg, torch.from_numpy(z["policy_avg"]))
    assert torch.equal(o.values_avg, torch.from_numpy(z["values_avg"]))
    ex, _ = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["exploitability"]))


def test_oracle_standard_cfr_bit_exact(golden_dir):
    z = np.load(os.path.join(golden_dir, "cfr_standard_cap2_t16.npz"))
    t = _build(z["pot"], z["stack"], int(z["cap"]), int(z["max_depth"]))
    o = ocfr.SubgameOracle(t.oracle_dict(z["boards"].astype(np.int64)), torch.from_numpy(z["ranges"]),
                           iterations=int(z["iterations"]), cfr_type="standard").solve()
    assert torch.equal(o.regrets, torch.from_numpy(z["regrets"]))
    assert torch.equal(o.weight_sums, torch.from_numpy(z["weight_sums"]))
    assert torch.equal(o.policy_avg, torch.from_numpy(z["policy_avg"]))
    assert torch.equal(o.values_avg[: o.N], torch.from_numpy(z["root_values"]))
    ex, _ = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["exploitability"]))


def test_oracle_zero_sum_value_targets_bit_exact(golden_dir):
    z = np.load(os.path.join(golden_dir, "cfr_zero_sum.npz"))
    cap, depth = int(z["cap"]), int(z["max_depth"])
    t = _build(z["river_pot"], z["river_stack"], cap, depth)
    o = ocfr.SubgameOracle(t.oracle_dict(z["river_boards"].astype(np.int64)), torch.from_numpy(z["river_ranges"]),
                           iterations=int(z["river_iterations"]), enforce_zero_sum=True).solve()
    assert torch.equal(o.policy_avg, torch.from_numpy(z["river_policy_avg"]))
    assert torch.equal(o.values_avg, torch.from_numpy(z["river_values_avg"]))
    # turn subgames: the leaves the model values are shifted too, and the best responses start from them
    t = _build(z["turn_pot"], z["turn_stack"], cap, depth, street=2)
    assert t.total_nodes == int(z["turn_total_nodes"])
    boards = np.concatenate([z["turn_boards"].astype(np.int64), np.full((z["turn_boards"].shape[0], 1), -1)], axis=1)
    model_nodes = np.nonzero(z["turn_model_mask"])[0]
    leaf_fn = pot_echo_leaf_fn(t, model_nodes, torch.from_numpy(z["hand_weights"]))
    o = ocfr.SubgameOracle(t.oracle_dict(boards), torch.from_numpy(z["turn_ranges"]),
                           iterations=int(z["turn_iterations"]), enforce_zero_sum=True,
                           leaf_fn=lambda b, idx: leaf_fn(b)).solve()
    assert torch.equal(o.policy_avg, torch.from_numpy(z["turn_policy_avg"]))
    assert torch.equal(o.values_avg, torch.from_numpy(z["turn_values_avg"]))
    ex, br = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["turn_exploitability"]))
    assert torch.equal(br, torch.from_numpy(z["turn_br_values"]))


def test_iteration_scalars_follow_the_schedules():
    """The host table the kernels read equals what the oracle (pinned to upstream above) computes
    per iteration, including a negative beta after a warm start."""
    T, ws, delay = 40, 15, 24
    sc = solver.iteration_scalars(T, cfr_type="discounted_plus", alpha=2.0, alpha_final=4.0, beta=-1.0,
                                  beta_final=-2.0, gamma=5.0, gamma_final=0.0, dcfr_delay=delay,
                                  warm_start_iterations=ws)

    class Sched:
        pass

    o = Sched()
    o.iterations, o.warm_start_iterations = T, ws
    o.alpha0, o.beta0, o.gamma0 = 2.0, -1.0, 5.0
    o.alpha_final, o.beta_final, o.gamma_final = 4.0, -2.0, 0.0
    for t in range(ws, T):
        ocfr.SubgameOracle.apply_schedules(o, t)
        assert sc[t]["num_pos"] == np.float32(t ** o.alpha) and sc[t]["den_pos"] == np.float32(t ** o.alpha + 1)
        assert sc[t]["num_neg"] == np.float32(t ** o.beta) and sc[t]["den_neg"] == np.float32(t ** o.beta + 1)
        assert sc[t]["do_mix"] == (1 if t > delay else 0)
        if t > delay:
            assert (sc[t]["mix_old"], sc[t]["mix_new"]) == (t - delay, 2)
    assert (sc[:ws]["do_mix"] == 0).all() and (sc[:ws]["num_neg"] == 1).all()
    # plain DCFR keeps its values (t = 0: 0**0 = 1, 0**1.5 = 0)
    plain = solver.iteration_scalars(4)
    assert plain[0]["num_pos"] == 0 and plain[0]["num_neg"] == 1 and plain[0]["do_mix"] == 0
    assert plain[3]["mix_old"] == 9 and plain[3]["mix_new"] == 16
    # standard CFR: no discount, weights (t, 1)
    std = solver.iteration_scalars(4, cfr_type="standard")
    assert std[2]["num_pos"] == 1 and std[2]["den_pos"] == 1 and (std[2]["mix_old"], std[2]["mix_new"]) == (2, 1)


def test_oracle_cfr_avg_bit_exact(golden_dir):
    """cfr_avg = True upstream: showdown values and regret weights at the beliefs under the average
    policy (river), model values de-averaged from the second iteration on and shifted to zero sum (turn)."""
    z = np.load(os.path.join(golden_dir, "cfr_avg.npz"))
    cap, depth = int(z["cap"]), int(z["max_depth"])
    t = _build(z["river_pot"], z["river_stack"], cap, depth)
    assert t.total_nodes == int(z["river_total_nodes"])
    o = ocfr.SubgameOracle(t.oracle_dict(z["river_boards"].astype(np.int64)), torch.from_numpy(z["river_ranges"]),
                           iterations=int(z["river_iterations"]), enforce_zero_sum=True, cfr_avg=True).solve()
    assert torch.equal(o.regrets, torch.from_numpy(z["river_regrets"]))
    assert torch.equal(o.policy_avg, torch.from_numpy(z["river_policy_avg"]))
    assert torch.equal(o.values_avg, torch.from_numpy(z["river_values_avg"]))
    # the flag matters: without it the regrets differ
    plain = ocfr.SubgameOracle(t.oracle_dict(z["river_boards"].astype(np.int64)), torch.from_numpy(z["river_ranges"]),
                               iterations=int(z["river_iterations"]), enforce_zero_sum=True).solve()
    assert not torch.equal(plain.regrets, o.regrets)
    t = _build(z["turn_pot"], z["turn_stack"], cap, depth, street=2)
    assert t.total_nodes == int(z["turn_total_nodes"])
    boards = np.concatenate([z["turn_boards"].astype(np.int64), np.full((z["turn_boards"].shape[0], 1), -1)], axis=1)
    model_nodes = np.nonzero(z["turn_model_mask"])[0]
    leaf_fn = pot_echo_leaf_fn(t, model_nodes, torch.from_numpy(z["hand_weights"]))
    o = ocfr.SubgameOracle(t.oracle_dict(boards), torch.from_numpy(z["turn_ranges"]),
                           iterations=int(z["turn_iterations"]), enforce_zero_sum=True, cfr_avg=True,
                           leaf_fn=lambda b, idx: leaf_fn(b)).solve()
    assert torch.equal(o.regrets, torch.from_numpy(z["turn_regrets"]))
    assert torch.equal(o.policy_avg, torch.from_numpy(z["turn_policy_avg"]))
    assert torch.equal(o.values_avg, torch.from_numpy(z["turn_values_avg"]))
    ex, br = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["turn_exploitability"]))
    assert torch.equal(br, torch.from_numpy(z["turn_br_values"]))


def test_oracle_running_value_average_bit_exact(golden_dir):
    """value_targets_from_final_policy = False upstream: values_avg is the running mix of the per-iteration
    values, shifted to zero sum every iteration; there is no final pass."""
    z = np.load(os.path.join(golden_dir, "cfr_running_values.npz"))
    cap, depth = int(z["cap"]), int(z["max_depth"])
    t = _build(z["river_pot"], z["river_stack"], cap, depth)
    assert t.total_nodes == int(z["river_total_nodes"])
    o = ocfr.SubgameOracle(t.oracle_dict(z["river_boards"].astype(np.int64)), torch.from_numpy(z["river_ranges"]),
                           iterations=int(z["river_iterations"]), enforce_zero_sum=True, final_policy_values=False).solve()
    assert torch.equal(o.policy_avg, torch.from_numpy(z["river_policy_avg"]))
    assert torch.equal(o.values_avg, torch.from_numpy(z["river_values_avg"]))
    ex, br = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["river_exploitability"]))
    assert torch.equal(br, torch.from_numpy(z["river_br_values"]))
    t = _build(z["turn_pot"], z["turn_stack"], cap, depth, street=2)
    assert t.total_nodes == int(z["turn_total_nodes"])
    boards = np.concatenate([z["turn_boards"].astype(np.int64), np.full((z["turn_boards"].shape[0], 1), -1)], axis=1)
    model_nodes = np.nonzero(z["turn_model_mask"])[0]
    leaf_fn = pot_echo_leaf_fn(t, model_nodes, torch.from_numpy(z["hand_weights"]))
    o = ocfr.SubgameOracle(t.oracle_dict(boards), torch.from_numpy(z["turn_ranges"]),
                           iterations=int(z["turn_iterations"]), enforce_zero_sum=True, final_policy_values=False,
                           leaf_fn=lambda b, idx: leaf_fn(b)).solve()
    assert torch.equal(o.policy_avg, torch.from_numpy(z["turn_policy_avg"]))
    assert torch.equal(o.values_avg, torch.from_numpy(z["turn_values_avg"]))
    ex, br = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["turn_exploitability"]))
    assert torch.equal(br, torch.from_numpy(z["turn_br_values"]))


def test_oracle_model_br_warm_start_bit_exact(golden_dir):
    """Warm start of type `model_br`: regrets seeded with iterations x multiplier x the regrets of not playing a
    best response against the start policy, on river subgames and on turn subgames with a stand-in model."""
    z = np.load(os.path.join(golden_dir, "cfr_warm_br.npz"))
    cap, depth, T, ws = int(z["cap"]), int(z["max_depth"]), int(z["iterations"]), int(z["warm_start_iterations"])
    for tag, street in (("river", 3), ("turn", 2)):
        t = _build(z[f"{tag}_pot"], z[f"{tag}_stack"], cap, depth, street=street)
        assert t.total_nodes == int(z[f"{tag}_total_nodes"])
        boards = z[f"{tag}_boards"].astype(np.int64)
        if boards.shape[1] < 5:
            boards = np.concatenate([boards, np.full((boards.shape[0], 5 - boards.shape[1]), -1)], axis=1)
        leaf = None
        if street == 2:
            fn = pot_echo_leaf_fn(t, np.nonzero(z["turn_model_mask"])[0], torch.from_numpy(z["hand_weights"]))
            leaf = lambda b, idx, fn=fn: fn(b)  # noqa: E731
        o = ocfr.SubgameOracle(t.oracle_dict(boards), torch.from_numpy(z[f"{tag}_ranges"]), iterations=T,
                               start_policy=torch.from_numpy(z[f"{tag}_start_policy"]), warm_start_iterations=ws,
                               warm_start_multiplier=float(z["warm_start_multiplier"]), warm_start_type="model_br",
                               leaf_fn=leaf)
        o.initialize()
        o.warm_start()
        assert torch.equal(o.regrets, torch.from_numpy(z[f"{tag}_seeded_regrets"]))
        for it in range(ws, T):
            o.iteration(it)
        o.finalize()
        assert torch.equal(o.policy_avg, torch.from_numpy(z[f"{tag}_policy_avg"]))
        assert torch.equal(o.values_avg[: o.N], torch.from_numpy(z[f"{tag}_root_values"]))
        ex, _ = o.exploitability()
        assert torch.equal(ex, torch.from_numpy(z[f"{tag}_exploitability"]))


def test_oracle_linear_cfr_bit_exact(golden_dir):
    z = np.load(os.path.join(golden_dir, "cfr_linear_cap2_t13.npz"))
    t = _build(z["pot"], z["stack"], int(z["cap"]), int(z["max_depth"]))
    o = ocfr.SubgameOracle(t.oracle_dict(z["boards"].astype(np.int64)), torch.from_numpy(z["ranges"]),
                           iterations=int(z["iterations"]), cfr_type="linear", cfr_plus=True).solve()
    assert torch.equal(o.regrets, torch.from_numpy(z["regrets"]))
    assert torch.equal(o.weight_sums, torch.from_numpy(z["weight_sums"]))
    assert torch.equal(o.policy_avg, torch.from_numpy(z["policy_avg"]))
    assert torch.equal(o.values_avg[: o.N], torch.from_numpy(z["root_values"]))
    ex, _ = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["exploitability"]))


def _defaults_case(z, tag, street):
    cap, depth = int(z["cap"]), int(z["max_depth"])
    t = _build(z[f"{tag}_pot"], z[f"{tag}_stack"], cap, depth, street=street)
    assert t.total_nodes == int(z[f"{tag}_total_nodes"])
    boards = z[f"{tag}_boards"].astype(np.int64)
    if boards.shape[1] < 5:
        boards = np.concatenate([boards, np.full((boards.shape[0], 5 - boards.shape[1]), -1)], axis=1)
    return t, boards


def test_oracle_dataclass_default_search_settings_bit_exact(golden_dir):
    """Everything a bare SearchConfig() switches on, together: linear CFR + CFR+ clamp, cfr_avg, running value
    averages, warm start of type model_br, zero-sum model."""
    z = np.load(os.path.join(golden_dir, "cfr_dataclass_defaults.npz"))
    T, ws = int(z["iterations"]), int(z["warm_start_iterations"])
    for tag, street in (("river", 3), ("turn", 2)):
        t, boards = _defaults_case(z, tag, street)
        leaf = None
        if street == 2:
            fn = pot_echo_leaf_fn(t, np.nonzero(z["turn_model_mask"])[0], torch.from_numpy(z["hand_weights"]))
            leaf = lambda b, idx, fn=fn: fn(b)  # noqa: E731
        o = ocfr.SubgameOracle(t.oracle_dict(boards), torch.from_numpy(z[f"{tag}_ranges"]), iterations=T,
                               cfr_type="linear", cfr_plus=True, cfr_avg=True, final_policy_values=False,
                               enforce_zero_sum=True, start_policy=torch.from_numpy(z[f"{tag}_start_policy"]),
                               warm_start_iterations=ws, warm_start_multiplier=float(z["warm_start_multiplier"]),
                               warm_start_type="model_br", leaf_fn=leaf).solve()
        assert torch.equal(o.regrets, torch.from_numpy(z[f"{tag}_regrets"]))
        assert torch.equal(o.policy_avg, torch.from_numpy(z[f"{tag}_policy_avg"]))
        assert torch.equal(o.values_avg[: o.N], torch.from_numpy(z[f"{tag}_root_values"]))
        ex, _ = o.exploitability()
        assert torch.equal(ex, torch.from_numpy(z[f"{tag}_exploitability"]))


def test_oracle_policy_delta_statistics_bit_exact(golden_dir):
    """`cfr_delta.*` of `_record_stats` (cfr_evaluator.py:1573-1605): the same keys (two of the five points
    fall on one iteration in the three-iteration solve) and the same fp32 values as upstream records."""
    z = np.load(os.path.join(golden_dir, "cfr_policy_delta.npz"))
    cap, depth = int(z["cap"]), int(z["max_depth"])
    for tag in ("plain", "short", "warm"):
        t = _build(z[f"{tag}_pot"], z[f"{tag}_stack"], cap, depth)
        assert t.total_nodes == int(z[f"{tag}_total_nodes"])
        ws = int(z[f"{tag}_warm_start_iterations"])
        kw = {}
        if ws:
            kw = dict(start_policy=torch.from_numpy(z[f"{tag}_start_policy"]), warm_start_iterations=ws,
                      warm_start_multiplier=float(z["warm_start_multiplier"]))
        o = ocfr.SubgameOracle(t.oracle_dict(z[f"{tag}_boards"].astype(np.int64)), torch.from_numpy(z[f"{tag}_ranges"]),
                               iterations=int(z[f"{tag}_iterations"]), **kw).solve()
        ex, _ = o.exploitability()
        assert torch.equal(ex, torch.from_numpy(z[f"{tag}_exploitability"]))
        keys = [f"cfr_delta.{int(q)}" for q in z[f"{tag}_delta_keys"]]
        assert sorted(o.stats) == sorted(keys)
        for k, want in zip(keys, z[f"{tag}_delta_values"]):
            assert o.stats[k] == want, (tag, k, o.stats[k], want)


def test_policy_delta_host_computation_against_the_oracle(golden_dir):
    """`stats.PolicyDelta` (what the evaluator records `cfr_delta.*` with) on the CPU: fed the oracle's
    regrets on either side of the recorded iterations, in the solver's row order."""
    from poker2_b200 import solver, stats as pstats

    z = np.load(os.path.join(golden_dir, "cfr_policy_delta.npz"))
    tag = "plain"
    t = _build(z[f"{tag}_pot"], z[f"{tag}_stack"], int(z["cap"]), int(z["max_depth"]))
    boards = z[f"{tag}_boards"].astype(np.int64)
    T = int(z[f"{tag}_iterations"])
    layout = solver.device_layout(t, boards)
    pd = pstats.PolicyDelta(t, boards, layout, "cpu")
    order = torch.from_numpy(np.ascontiguousarray(layout.to_level_major)).long()
    rows = lambda x: solver.pad_rows(x[order])  # noqa: E731  upstream node order -> solver rows
    points = pstats.delta_checkpoints(0, T)
    assert points == {0: 0, 2: 25, 4: 50, 6: 75, 8: 100}
    assert pstats.delta_checkpoints(0, 3) == {0: 0, 1: 50, 2: 75}
    assert pstats.delta_checkpoints(3, 10) == {3: 0, 4: 25, 6: 50, 8: 75, 9: 100}  # 4.5 and 7.5 round to even
    o = ocfr.SubgameOracle(t.oracle_dict(boards), torch.from_numpy(z[f"{tag}_ranges"]), iterations=T)
    o.initialize()
    for it in range(T):
        before = pd.start_policy(None) if it == 0 else pd.policy_of(rows(o.regrets))
        o.iteration(it)
        if it in points:
            got = float(pd(before, pd.policy_of(rows(o.regrets))))
            assert got == pytest.approx(o.stats[f"cfr_delta.{points[it]}"], rel=1e-6), it
    assert len(o.stats) == 5


def test_oracle_on_the_production_tree_shape_bit_exact(golden_dir):
    """Depth 5, bet sizes {0.5, 1.0}, no raise cap, deep stacks: the trees of the production search settings
    (273 and 242 nodes), leaves valued by the stand-in model, against the upstream run."""
    z = np.load(os.path.join(golden_dir, "cfr_depth5_nocap_t6.npz"))
    t = ptree.build_trees(ptree.root_states(z["pot"], z["stack"], min_raise=2, street=2), BET_BINS, int(z["max_depth"]), bb=2)
    assert t.total_nodes == int(z["total_nodes"]) and np.bincount(t.root_of).tolist() == [273, 242]
    assert np.array_equal(t.leaf_mask & ~t.state.done, z["model_mask"])
    boards = np.concatenate([z["boards"].astype(np.int64), np.full((2, 1), -1)], axis=1)
    w = torch.from_numpy(z["hand_weights"])
    o = ocfr.SubgameOracle(t.oracle_dict(boards), torch.from_numpy(z["ranges"]), iterations=int(z["iterations"]),
                           leaf_fn=lambda b, idx: pot_echo_leaf_fn(t, idx, w)(b)).solve()
    rows = torch.from_numpy(z["rows"])
    assert torch.equal(o.policy_avg[rows], torch.from_numpy(z["policy_avg_rows"]))
    assert torch.equal(o.regrets[rows], torch.from_numpy(z["regrets_rows"]))
    assert torch.equal(o.values_avg[:2], torch.from_numpy(z["root_values"]))
    ex, br = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["exploitability"])) and torch.equal(br, torch.from_numpy(z["br_values"]))


def test_oracle_with_the_default_bet_sizes_bit_exact(golden_dir):
    """Eight actions per node (the bet sizes of the upstream dataclass) at depth 3 without a raise cap, leaves at
    the depth limit valued by the stand-in model: trees of 280 and 143 nodes against the upstream run."""
    z = np.load(os.path.join(golden_dir, "cfr_default_bins_depth3_t6.npz"))
    bins = [float(x) for x in z["bet_bins"]]
    t = ptree.build_trees(ptree.root_states(z["pot"], z["stack"], min_raise=2), bins, int(z["max_depth"]), bb=2)
    assert t.total_nodes == int(z["total_nodes"]) and t.num_actions == 8 and int(t.child_count.max()) == 8
    assert np.array_equal(t.leaf_mask & ~t.state.done, z["model_mask"])
    boards = z["boards"].astype(np.int64)
    w = torch.from_numpy(z["hand_weights"])
    o = ocfr.SubgameOracle(t.oracle_dict(boards), torch.from_numpy(z["ranges"]), iterations=int(z["iterations"]),
                           leaf_fn=lambda b, idx: pot_echo_leaf_fn(t, idx, w)(b)).solve()
    rows = torch.from_numpy(z["rows"])
    assert torch.equal(o.policy_avg[rows], torch.from_numpy(z["policy_avg_rows"]))
    assert torch.equal(o.regrets[rows], torch.from_numpy(z["regrets_rows"]))
    assert torch.equal(o.values_avg[:2], torch.from_numpy(z["root_values"]))
    ex, br = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["exploitability"])) and torch.equal(br, torch.from_numpy(z["br_values"]))

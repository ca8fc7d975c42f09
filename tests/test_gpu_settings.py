"""The CUDA solver under settings beyond plain DCFR, against arrays produced by the upstream
evaluator: the production search block, standard CFR, zero-sum value targets, and the headline
workload at depth (16 ragged roots x 256 iterations)."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-6  # fp32 strategies and values: 1e-5 relative plus a small absolute term near zero


def _close(name, got, want, rtol=RTOL, atol=ATOL):
    err = (got - want).abs()
    print(f"{name}: max abs {err.max().item():.3e}")
    torch.testing.assert_close(got, want, rtol=rtol, atol=atol)


def test_production_search_block_matches_upstream(cuda_device, golden_dir):
    """discounted_plus with a delay, exponent schedules (alpha 2->4, beta -1->-2, gamma 5->0), warm
    start of type `model` (15 iterations, multiplier 10), zero-sum value targets: the search block of
    the upstream production configuration at a reduced iteration count."""
    from poker2_b200 import solver, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_production_cap2_t40.npz"))
    T, ws, delay = int(z["iterations"]), int(z["warm_start_iterations"]), int(z["dcfr_delay"])
    trees = ptree.build_trees(ptree.root_states(z["pot"], z["stack"], min_raise=2), [0.5, 1.0], int(z["max_depth"]),
                              bb=2, max_raises=int(z["cap"]))
    assert trees.total_nodes == int(z["total_nodes"])
    boards = z["boards"].astype(np.int64)
    layout = solver.device_layout(trees, boards)
    sv = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True, sampling=True)
    sv.set_sampling_schedule(torch.from_numpy(z["t_sample"]), warm_start_iterations=ws)
    rb = solver.pad_rows(torch.from_numpy(z["ranges"]).to(cuda_device)).contiguous()
    kw = dict(cfr_type="discounted_plus", gamma=float(z["gamma"][0]), dcfr_delay=delay)
    scal = solver.iteration_scalars(T, alpha=float(z["alpha"][0]), alpha_final=float(z["alpha"][1]),
                                    beta=float(z["beta"][0]), beta_final=float(z["beta"][1]),
                                    gamma_final=float(z["gamma"][1]), warm_start_iterations=ws, **kw)
    first = solver.warm_start_mix_scalars(scal, warm_start_iterations=ws, **kw)
    res = sv.solve(rb, scal, start_policy=torch.from_numpy(z["start_policy"]), warm_start_iterations=ws,
                   warm_start_multiplier=float(z["warm_start_multiplier"]), warm_start_scalars=first,
                   enforce_zero_sum=True)
    assert sv.status() == 0
    n = trees.num_roots
    for name, got in [("regrets", res.regrets), ("weight_sums", res.weight_sums), ("policy_avg", res.policy_avg),
                      ("policy_sample", res.policy_sample)]:
        _close(name, res.level_major(got).cpu()[n:], torch.from_numpy(z[name])[n:])
    _close("root_values", res.root_values[..., :1326].cpu(), torch.from_numpy(z["root_values"]))
    _close("values_avg", res.level_major(res.values_avg).cpu(), torch.from_numpy(z["values_avg"]))
    _close("exploitability", res.exploitability.cpu(), torch.from_numpy(z["exploitability"]), rtol=1e-4)


def test_standard_cfr_matches_upstream(cuda_device, golden_dir):
    from poker2_b200 import solver

    z = np.load(os.path.join(golden_dir, "cfr_standard_cap2_t16.npz"))
    res, trees = solver.solve_subgames(z["boards"].astype(np.int64), torch.from_numpy(z["ranges"]), z["pot"], z["stack"],
                                       iterations=int(z["iterations"]), max_depth=int(z["max_depth"]),
                                       max_raises=int(z["cap"]), cfr_type="standard", exploitability=True,
                                       device=cuda_device)
    assert trees.total_nodes == int(z["total_nodes"])
    n = trees.num_roots
    for name, got in [("regrets", res.regrets), ("weight_sums", res.weight_sums), ("policy_avg", res.policy_avg)]:
        _close(name, res.level_major(got).cpu()[n:], torch.from_numpy(z[name])[n:])
    _close("root_values", res.root_values[..., :1326].cpu(), torch.from_numpy(z["root_values"]))
    _close("exploitability", res.exploitability.cpu(), torch.from_numpy(z["exploitability"]), rtol=1e-4)


def test_zero_sum_value_targets_match_upstream(cuda_device, golden_dir):
    """`model.enforce_zero_sum = True` upstream: every node's final values minus the mean over the
    players of sum_h values * beliefs_avg, except at terminal nodes.  River subgames through the
    one-call solve; turn subgames (leaves valued by a stand-in model, shifted too) pass by pass."""
    from leaf_models import pot_echo_leaf_fn
    from poker2_b200 import solver, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_zero_sum.npz"))
    cap, depth = int(z["cap"]), int(z["max_depth"])
    res, trees = solver.solve_subgames(z["river_boards"].astype(np.int64), torch.from_numpy(z["river_ranges"]),
                                       z["river_pot"], z["river_stack"], iterations=int(z["river_iterations"]),
                                       max_depth=depth, max_raises=cap, keep_node_values=True, exploitability=True,
                                       enforce_zero_sum=True, device=cuda_device)
    assert trees.total_nodes == int(z["river_total_nodes"])
    n = trees.num_roots
    _close("river policy_avg", res.level_major(res.policy_avg).cpu()[n:], torch.from_numpy(z["river_policy_avg"])[n:])
    _close("river values_avg", res.level_major(res.values_avg).cpu(), torch.from_numpy(z["river_values_avg"]))
    _close("river root_values", res.root_values[..., :1326].cpu(), torch.from_numpy(z["river_values_avg"])[:n])
    _close("river exploitability", res.exploitability.cpu(), torch.from_numpy(z["river_exploitability"]), rtol=1e-4)
    # without the flag the root values differ from the shifted ones (the test would notice a no-op)
    plain, _ = solver.solve_subgames(z["river_boards"].astype(np.int64), torch.from_numpy(z["river_ranges"]),
                                     z["river_pot"], z["river_stack"], iterations=int(z["river_iterations"]),
                                     max_depth=depth, max_raises=cap, device=cuda_device)
    assert (plain.root_values[..., :1326].cpu() - torch.from_numpy(z["river_values_avg"])[:n]).abs().max() > 1e-4

    roots = ptree.root_states(z["turn_pot"], z["turn_stack"], min_raise=2, street=2)
    trees = ptree.build_trees(roots, [0.5, 1.0], depth, bb=2, max_raises=cap)
    assert trees.total_nodes == int(z["turn_total_nodes"])
    boards = np.concatenate([z["turn_boards"].astype(np.int64), np.full((z["turn_boards"].shape[0], 1), -1)], axis=1)
    layout = solver.device_layout(trees, boards)
    sv = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True)
    leaf_fn = pot_echo_leaf_fn(trees, layout.model_nodes, torch.from_numpy(z["hand_weights"]))
    rb = solver.pad_rows(torch.from_numpy(z["turn_ranges"]).to(cuda_device)).contiguous()
    res = sv.solve(rb, solver.iteration_scalars(int(z["turn_iterations"])), leaf_fn, enforce_zero_sum=True)
    n = trees.num_roots
    _close("turn policy_avg", res.level_major(res.policy_avg).cpu()[n:], torch.from_numpy(z["turn_policy_avg"])[n:])
    _close("turn values_avg", res.level_major(res.values_avg).cpu(), torch.from_numpy(z["turn_values_avg"]))
    _close("turn exploitability", res.exploitability.cpu(), torch.from_numpy(z["turn_exploitability"]), rtol=1e-4)
    _close("turn br_values", res.br_values.cpu(), torch.from_numpy(z["turn_br_values"]), rtol=1e-4)


def test_ragged_roots_at_256_iterations_match_upstream(cuda_device, golden_dir):
    """The headline configuration at depth: 16 ragged river roots (pot U[20,200], stack U[100,1000]),
    256 DCFR iterations, against the upstream run: root values, exploitability and a fixed subsample
    of the average-policy and regret rows."""
    from poker2_b200 import solver

    z = np.load(os.path.join(golden_dir, "cfr_ragged16_cap2_t256.npz"))
    res, trees = solver.solve_subgames(z["boards"].astype(np.int64), torch.from_numpy(z["ranges"]), z["pot"], z["stack"],
                                       iterations=int(z["iterations"]), max_depth=int(z["max_depth"]),
                                       max_raises=int(z["cap"]), exploitability=True, device=cuda_device)
    assert trees.total_nodes == int(z["total_nodes"])
    rows = torch.from_numpy(z["policy_rows"])
    _close("policy_avg rows", res.level_major(res.policy_avg).cpu()[rows], torch.from_numpy(z["policy_avg_rows"]))
    _close("regret rows", res.level_major(res.regrets).cpu()[rows], torch.from_numpy(z["regret_rows"]))
    _close("root_values", res.root_values[..., :1326].cpu(), torch.from_numpy(z["root_values"]))
    _close("exploitability", res.exploitability.cpu(), torch.from_numpy(z["exploitability"]), rtol=1e-4)
    _close("br_values", res.br_values.cpu(), torch.from_numpy(z["br_values"]), rtol=1e-4)


def test_cfr_avg_matches_upstream(cuda_device, golden_dir):
    """`cfr_avg = True` upstream (the dataclass default): showdown values and regret weights at the beliefs
    under the average policy.  River subgames through the one-call solve; turn subgames pass by pass, the
    stand-in model seeing the average beliefs and its values de-averaged from the second iteration on."""
    from leaf_models import pot_echo_leaf_fn
    from poker2_b200 import solver, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_avg.npz"))
    cap, depth = int(z["cap"]), int(z["max_depth"])
    res, trees = solver.solve_subgames(z["river_boards"].astype(np.int64), torch.from_numpy(z["river_ranges"]),
                                       z["river_pot"], z["river_stack"], iterations=int(z["river_iterations"]),
                                       max_depth=depth, max_raises=cap, keep_node_values=True, exploitability=True,
                                       enforce_zero_sum=True, cfr_avg=True, device=cuda_device)
    assert trees.total_nodes == int(z["river_total_nodes"])
    n = trees.num_roots
    _close("river regrets", res.level_major(res.regrets).cpu()[n:], torch.from_numpy(z["river_regrets"])[n:])
    _close("river policy_avg", res.level_major(res.policy_avg).cpu()[n:], torch.from_numpy(z["river_policy_avg"])[n:])
    _close("river values_avg", res.level_major(res.values_avg).cpu(), torch.from_numpy(z["river_values_avg"]))
    _close("river exploitability", res.exploitability.cpu(), torch.from_numpy(z["river_exploitability"]), rtol=1e-4)
    # the flag matters: without it the regrets differ visibly
    plain, _ = solver.solve_subgames(z["river_boards"].astype(np.int64), torch.from_numpy(z["river_ranges"]),
                                     z["river_pot"], z["river_stack"], iterations=int(z["river_iterations"]),
                                     max_depth=depth, max_raises=cap, device=cuda_device)
    assert (plain.level_major(plain.regrets).cpu() - torch.from_numpy(z["river_regrets"])).abs().max() > 1e-4

    roots = ptree.root_states(z["turn_pot"], z["turn_stack"], min_raise=2, street=2)
    trees = ptree.build_trees(roots, [0.5, 1.0], depth, bb=2, max_raises=cap)
    assert trees.total_nodes == int(z["turn_total_nodes"])
    boards = np.concatenate([z["turn_boards"].astype(np.int64), np.full((z["turn_boards"].shape[0], 1), -1)], axis=1)
    layout = solver.device_layout(trees, boards)
    sv = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True)
    leaf_fn = pot_echo_leaf_fn(trees, layout.model_nodes, torch.from_numpy(z["hand_weights"]))
    rb = solver.pad_rows(torch.from_numpy(z["turn_ranges"]).to(cuda_device)).contiguous()
    res = sv.solve(rb, solver.iteration_scalars(int(z["turn_iterations"])), leaf_fn, enforce_zero_sum=True, cfr_avg=True)
    assert sv.status() == 0
    n = trees.num_roots
    _close("turn regrets", res.level_major(res.regrets).cpu()[n:], torch.from_numpy(z["turn_regrets"])[n:])
    _close("turn policy_avg", res.level_major(res.policy_avg).cpu()[n:], torch.from_numpy(z["turn_policy_avg"])[n:])
    _close("turn values_avg", res.level_major(res.values_avg).cpu(), torch.from_numpy(z["turn_values_avg"]))
    _close("turn exploitability", res.exploitability.cpu(), torch.from_numpy(z["turn_exploitability"]), rtol=1e-4)
    _close("turn br_values", res.br_values.cpu(), torch.from_numpy(z["turn_br_values"]), rtol=1e-4)


def test_running_value_average_matches_upstream(cuda_device, golden_dir):
    """`value_targets_from_final_policy = False` upstream: the value outputs are the running mix of the
    per-iteration node values, shifted to zero sum every iteration; the best responses start from those
    averages at the leaves.  River and turn subgames, pass by pass."""
    from leaf_models import pot_echo_leaf_fn
    from poker2_b200 import solver, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_running_values.npz"))
    cap, depth = int(z["cap"]), int(z["max_depth"])
    for street, tag in ((3, "river"), (2, "turn")):
        roots = ptree.root_states(z[f"{tag}_pot"], z[f"{tag}_stack"], min_raise=2, street=street)
        trees = ptree.build_trees(roots, [0.5, 1.0], depth, bb=2, max_raises=cap)
        assert trees.total_nodes == int(z[f"{tag}_total_nodes"])
        boards = z[f"{tag}_boards"].astype(np.int64)
        if boards.shape[1] < 5:
            boards = np.concatenate([boards, np.full((boards.shape[0], 5 - boards.shape[1]), -1)], axis=1)
        layout = solver.device_layout(trees, boards)
        sv = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True)
        leaf_fn = None
        if street == 2:
            leaf_fn = pot_echo_leaf_fn(trees, layout.model_nodes, torch.from_numpy(z["hand_weights"]))
        rb = solver.pad_rows(torch.from_numpy(z[f"{tag}_ranges"]).to(cuda_device)).contiguous()
        res = sv.solve(rb, solver.iteration_scalars(int(z[f"{tag}_iterations"])), leaf_fn, enforce_zero_sum=True,
                       running_values=True)
        assert sv.status() == 0
        n = trees.num_roots
        _close(f"{tag} policy_avg", res.level_major(res.policy_avg).cpu()[n:], torch.from_numpy(z[f"{tag}_policy_avg"])[n:])
        _close(f"{tag} values_avg", res.level_major(res.values_avg).cpu(), torch.from_numpy(z[f"{tag}_values_avg"]))
        _close(f"{tag} root_values", res.root_values[..., :1326].cpu(), torch.from_numpy(z[f"{tag}_values_avg"])[:n])
        _close(f"{tag} exploitability", res.exploitability.cpu(), torch.from_numpy(z[f"{tag}_exploitability"]), rtol=1e-4)
        _close(f"{tag} br_values", res.br_values.cpu(), torch.from_numpy(z[f"{tag}_br_values"]), rtol=1e-4)


def test_model_br_warm_start_matches_upstream(cuda_device, golden_dir):
    """Warm start of type `model_br` (the dataclass default upstream): after the start pass, a best-response
    pass against the start policy seeds the regrets; river subgames and turn subgames with a stand-in model."""
    from leaf_models import pot_echo_leaf_fn
    from poker2_b200 import solver, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_warm_br.npz"))
    cap, depth, T, ws = int(z["cap"]), int(z["max_depth"]), int(z["iterations"]), int(z["warm_start_iterations"])
    for tag, street in (("river", 3), ("turn", 2)):
        roots = ptree.root_states(z[f"{tag}_pot"], z[f"{tag}_stack"], min_raise=2, street=street)
        trees = ptree.build_trees(roots, [0.5, 1.0], depth, bb=2, max_raises=cap)
        assert trees.total_nodes == int(z[f"{tag}_total_nodes"])
        boards = z[f"{tag}_boards"].astype(np.int64)
        if boards.shape[1] < 5:
            boards = np.concatenate([boards, np.full((boards.shape[0], 5 - boards.shape[1]), -1)], axis=1)
        layout = solver.device_layout(trees, boards)
        sv = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True)
        leaf_fn = None
        if street == 2:
            leaf_fn = pot_echo_leaf_fn(trees, layout.model_nodes, torch.from_numpy(z["hand_weights"]))
        rb = solver.pad_rows(torch.from_numpy(z[f"{tag}_ranges"]).to(cuda_device)).contiguous()
        res = sv.solve(rb, solver.iteration_scalars(T, warm_start_iterations=ws), leaf_fn,
                       start_policy=torch.from_numpy(z[f"{tag}_start_policy"]), warm_start_iterations=ws,
                       warm_start_multiplier=float(z["warm_start_multiplier"]), warm_start_type="model_br")
        assert sv.status() == 0
        n = trees.num_roots
        _close(f"{tag} policy_avg", res.level_major(res.policy_avg).cpu()[n:], torch.from_numpy(z[f"{tag}_policy_avg"])[n:])
        _close(f"{tag} root_values", res.root_values[..., :1326].cpu(), torch.from_numpy(z[f"{tag}_root_values"]))
        _close(f"{tag} exploitability", res.exploitability.cpu(), torch.from_numpy(z[f"{tag}_exploitability"]), rtol=1e-4)
        # the seeding itself: one more solve that stops after the warm start's own policy update
        sv2 = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True)
        seen = {}
        orig = sv2._step

        def spy(root_beliefs, sc, iterations, flags, pb, pe, phases, orig=orig, sv2=sv2, seen=seen):
            orig(root_beliefs, sc, iterations, flags, pb, pe, phases)
            if phases == 8:
                seen["raw"] = sv2.regrets.clone()

        sv2._step = spy
        sv2.solve(rb, solver.iteration_scalars(T, warm_start_iterations=ws), leaf_fn,
                  start_policy=torch.from_numpy(z[f"{tag}_start_policy"]), warm_start_iterations=ws,
                  warm_start_multiplier=float(z["warm_start_multiplier"]), warm_start_type="model_br")
        weight = float(ws) * float(z["warm_start_multiplier"])
        order = solver.layout_tensor(layout, "from_level_major", cuda_device)
        seeded = (seen["raw"] * weight).index_select(0, order)[:, :1326].cpu()
        _close(f"{tag} seeded regrets", seeded[n:], torch.from_numpy(z[f"{tag}_seeded_regrets"])[n:])


def test_linear_cfr_matches_upstream(cuda_device, golden_dir):
    """cfr_type = linear with the CFR+ clamp: alternating updates, mixing weights (t, 2); every pass in the
    general kernel.  Through the one-call solve and through the allocation-free entry."""
    from poker2_b200 import solver

    z = np.load(os.path.join(golden_dir, "cfr_linear_cap2_t13.npz"))
    res, trees = solver.solve_subgames(z["boards"].astype(np.int64), torch.from_numpy(z["ranges"]), z["pot"], z["stack"],
                                       iterations=int(z["iterations"]), max_depth=int(z["max_depth"]),
                                       max_raises=int(z["cap"]), cfr_type="linear", cfr_plus=True, exploitability=True,
                                       device=cuda_device)
    assert trees.total_nodes == int(z["total_nodes"])
    n = trees.num_roots
    for name, got in [("regrets", res.regrets), ("weight_sums", res.weight_sums), ("policy_avg", res.policy_avg)]:
        _close(name, res.level_major(got).cpu()[n:], torch.from_numpy(z[name])[n:])
    _close("root_values", res.root_values[..., :1326].cpu(), torch.from_numpy(z["root_values"]))
    _close("exploitability", res.exploitability.cpu(), torch.from_numpy(z["exploitability"]), rtol=1e-4)


def test_production_search_block_through_the_one_call_solve(cuda_device, golden_dir):
    """The production search block (warm start of type `model`, discounted_plus with a delay, exponent
    schedules, zero-sum targets) through `SubgameSolver.solve`, whose iteration passes run in the lean
    kernel: same fixture as the stepped test above, and the same bits as the stepped solve."""
    from poker2_b200 import solver, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_production_cap2_t40.npz"))
    T, ws, delay = int(z["iterations"]), int(z["warm_start_iterations"]), int(z["dcfr_delay"])
    trees = ptree.build_trees(ptree.root_states(z["pot"], z["stack"], min_raise=2), [0.5, 1.0], int(z["max_depth"]),
                              bb=2, max_raises=int(z["cap"]))
    boards = z["boards"].astype(np.int64)
    layout = solver.device_layout(trees, boards)
    rb = solver.pad_rows(torch.from_numpy(z["ranges"]).to(cuda_device)).contiguous()
    kw = dict(cfr_type="discounted_plus", gamma=float(z["gamma"][0]), dcfr_delay=delay)
    scal = solver.iteration_scalars(T, alpha=float(z["alpha"][0]), alpha_final=float(z["alpha"][1]),
                                    beta=float(z["beta"][0]), beta_final=float(z["beta"][1]),
                                    gamma_final=float(z["gamma"][1]), warm_start_iterations=ws, **kw)
    first = solver.warm_start_mix_scalars(scal, warm_start_iterations=ws, **kw)
    args = dict(start_policy=torch.from_numpy(z["start_policy"]), warm_start_iterations=ws,
                warm_start_multiplier=float(z["warm_start_multiplier"]), warm_start_scalars=first, enforce_zero_sum=True)
    results = []
    for lean in (True, False):
        sv = solver.SubgameSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True, sampling=True,
                                  lean_iterations=lean)
        sv.set_sampling_schedule(torch.from_numpy(z["t_sample"]), warm_start_iterations=ws)
        res = sv.solve(rb, scal, check=True, **args) if lean else None
        if not lean:
            # the general kernel needs the larger scratch area for the hand-over between its two launches
            with pytest.raises(RuntimeError):
                sv.solve(rb, scal, **args)
            continue
        n = trees.num_roots
        for name, got in [("regrets", res.regrets), ("weight_sums", res.weight_sums), ("policy_avg", res.policy_avg),
                          ("policy_sample", res.policy_sample)]:
            _close(name, res.level_major(got).cpu()[n:], torch.from_numpy(z[name])[n:])
        _close("root_values", res.root_values[..., :1326].cpu(), torch.from_numpy(z["root_values"]))
        _close("values_avg", res.level_major(res.values_avg).cpu(), torch.from_numpy(z["values_avg"]))
        _close("exploitability", res.exploitability.cpu(), torch.from_numpy(z["exploitability"]), rtol=1e-4)
        results.append(res)
    stepped = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True, sampling=True)
    stepped.set_sampling_schedule(torch.from_numpy(z["t_sample"]), warm_start_iterations=ws)
    ref = stepped.solve(rb, scal, **args)
    for name in ("regrets", "weight_sums", "policy_avg", "root_values", "values_avg", "exploitability"):
        assert torch.equal(getattr(results[0], name), getattr(ref, name)), name


def test_dataclass_default_search_settings_match_upstream(cuda_device, golden_dir):
    """Everything a bare SearchConfig() switches on, together: linear CFR with the CFR+ clamp, cfr_avg, value
    targets from the running average, warm start of type model_br, zero-sum model; river and turn subgames."""
    from leaf_models import pot_echo_leaf_fn
    from poker2_b200 import solver, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_dataclass_defaults.npz"))
    cap, depth, T, ws = int(z["cap"]), int(z["max_depth"]), int(z["iterations"]), int(z["warm_start_iterations"])
    for tag, street in (("river", 3), ("turn", 2)):
        roots = ptree.root_states(z[f"{tag}_pot"], z[f"{tag}_stack"], min_raise=2, street=street)
        trees = ptree.build_trees(roots, [0.5, 1.0], depth, bb=2, max_raises=cap)
        assert trees.total_nodes == int(z[f"{tag}_total_nodes"])
        boards = z[f"{tag}_boards"].astype(np.int64)
        if boards.shape[1] < 5:
            boards = np.concatenate([boards, np.full((boards.shape[0], 5 - boards.shape[1]), -1)], axis=1)
        layout = solver.device_layout(trees, boards)
        sv = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True)
        leaf_fn = None
        if street == 2:
            leaf_fn = pot_echo_leaf_fn(trees, layout.model_nodes, torch.from_numpy(z["hand_weights"]))
        rb = solver.pad_rows(torch.from_numpy(z[f"{tag}_ranges"]).to(cuda_device)).contiguous()
        scal = solver.iteration_scalars(T, cfr_type="linear", warm_start_iterations=ws)
        first = solver.warm_start_mix_scalars(scal, cfr_type="linear", gamma=2.0, dcfr_delay=0, warm_start_iterations=ws)
        res = sv.solve(rb, scal, leaf_fn, cfr_plus=True, cfr_avg=True, running_values=True, enforce_zero_sum=True,
                       start_policy=torch.from_numpy(z[f"{tag}_start_policy"]), warm_start_iterations=ws,
                       warm_start_multiplier=float(z["warm_start_multiplier"]), warm_start_type="model_br",
                       warm_start_scalars=first)
        assert sv.status() == 0
        n = trees.num_roots
        # the best responses of the seeding add up in another fp64 order than the CPU's, and the clamped regret
        # matching that follows amplifies the last-bit differences: 1e-4 relative / 5e-6 absolute here (one policy
        # entry in 1.5e5 is 4e-5 off; the single settings are held to 1e-5 / 1e-6 by the tests above)
        tol = dict(rtol=1e-4, atol=5e-6)
        _close(f"{tag} regrets", res.level_major(res.regrets).cpu()[n:], torch.from_numpy(z[f"{tag}_regrets"])[n:], **tol)
        _close(f"{tag} policy_avg", res.level_major(res.policy_avg).cpu()[n:], torch.from_numpy(z[f"{tag}_policy_avg"])[n:],
               **tol)
        _close(f"{tag} root_values", res.root_values[..., :1326].cpu(), torch.from_numpy(z[f"{tag}_root_values"]), **tol)
        _close(f"{tag} exploitability", res.exploitability.cpu(), torch.from_numpy(z[f"{tag}_exploitability"]), rtol=1e-4)


def test_policy_delta_statistics_match_upstream(cuda_device, golden_dir):
    """`cfr_delta.*` (`_record_stats`, cfr_evaluator.py:1573-1605) from the regrets on either side of the five
    recorded iterations: a plain solve, a three-iteration solve (two of the five points fall together, so
    upstream writes three keys) and a solve warm-started from a policy head.  The sums behind the statistic
    run in another order than upstream's tensor reductions, hence 1e-5 relative."""
    from poker2_b200 import solver, stats as pstats, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_policy_delta.npz"))
    for tag in ("plain", "short", "warm"):
        T, ws = int(z[f"{tag}_iterations"]), int(z[f"{tag}_warm_start_iterations"])
        trees = ptree.build_trees(ptree.root_states(z[f"{tag}_pot"], z[f"{tag}_stack"], min_raise=2), [0.5, 1.0],
                                  int(z["max_depth"]), bb=2, max_raises=int(z["cap"]))
        assert trees.total_nodes == int(z[f"{tag}_total_nodes"])
        boards = z[f"{tag}_boards"].astype(np.int64)
        layout = solver.device_layout(trees, boards)
        sv = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True)
        rb = solver.pad_rows(torch.from_numpy(z[f"{tag}_ranges"]).to(cuda_device)).contiguous()
        scal = solver.iteration_scalars(T, warm_start_iterations=ws)
        kw = {}
        if ws:
            kw = dict(start_policy=torch.from_numpy(z[f"{tag}_start_policy"]), warm_start_iterations=ws,
                      warm_start_multiplier=float(z["warm_start_multiplier"]),
                      warm_start_scalars=solver.warm_start_mix_scalars(scal, cfr_type="discounted", gamma=2.0, dcfr_delay=0,
                                                                       warm_start_iterations=ws))
        res = sv.solve(rb, scal, policy_delta=pstats.PolicyDelta(trees, boards, layout, cuda_device), **kw)
        _close(f"{tag} exploitability", res.exploitability.cpu(), torch.from_numpy(z[f"{tag}_exploitability"]), rtol=1e-4)
        assert sorted(sv.policy_deltas) == [int(q) for q in z[f"{tag}_delta_keys"]]
        for q, want in zip(z[f"{tag}_delta_keys"], z[f"{tag}_delta_values"]):
            got = float(sv.policy_deltas[int(q)])
            print(f"{tag} cfr_delta.{int(q)}: {got:.8f} (upstream {want:.8f})")
            assert got == pytest.approx(float(want), rel=1e-5, abs=1e-7)

"""`step_evaluator.StepCFREvaluator`: the upstream evaluator's step methods on the step-level kernels, with the
state in the upstream layout.  Checked against a full upstream run, against the CPU oracle after every
single iteration, against the one-call solver, and on turn subgames with a stand-in leaf model."""
import os

import numpy as np
import pytest
import torch

from leaf_models import pot_echo_leaf_fn

pytestmark = pytest.mark.gpu

# Every step kernel rounds like the upstream CPU code (sums over hands in the order of its reduction, fp64 card
# sums, IEEE quotients), so the comparisons below are for equal bits; the solver's own kernels are held to the
# same standard elsewhere.


def _close(name, got, want):
    want = want if torch.is_tensor(want) else torch.from_numpy(want)
    diff = (got.cpu() - want).abs().max().item()
    print(f"{name}: max abs {diff:.3e}")
    assert torch.equal(got.cpu(), want), f"{name}: max abs difference {diff:.3e}"


def test_step_methods_reproduce_an_upstream_run(cuda_device, golden_dir):
    """Eight iterations driven through `evaluate_cfr`: every state tensor the upstream run left behind."""
    from poker2_b200 import step_evaluator, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_single_cap2_t8.npz"))
    trees = ptree.build_trees(ptree.root_states(z["pot"], z["stack"], min_raise=2), [0.5, 1.0], int(z["max_depth"]),
                              bb=2, max_raises=int(z["cap"]))
    assert trees.total_nodes == int(z["total_nodes"])
    ev = step_evaluator.StepCFREvaluator(trees, z["boards"].astype(np.int64), torch.from_numpy(z["ranges"]), cuda_device,
                                         iterations=int(z["iterations"]))
    ev.evaluate_cfr()
    n = trees.num_roots
    _close("policy_probs", ev.policy_probs[n:], z["policy"][n:])
    _close("policy_probs_avg", ev.policy_probs_avg[n:], z["policy_avg"][n:])
    _close("cumulative_regrets", ev.cumulative_regrets[n:], z["regrets"][n:])
    _close("regret_weight_sums", ev.regret_weight_sums[n:], z["weight_sums"][n:])
    _close("beliefs", ev.beliefs, z["beliefs"])
    _close("latest_values", ev.latest_values, z["latest_values"])
    _close("values_avg", ev.values_avg, z["values_avg"])


@pytest.mark.parametrize("cfr_type,cfr_plus", [("discounted", False), ("discounted_plus", True), ("standard", False)])
def test_every_iteration_against_the_oracle_and_the_solver(cuda_device, golden_dir, cfr_type, cfr_plus):
    """State after each `cfr_iteration(t)` against the CPU oracle's state after its iteration t (ragged roots, no
    resynchronisation in between), and the final state against the one-call solver."""
    from oracle import cfr as ocfr
    from poker2_b200 import solver, step_evaluator, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_batch_cap2_t24.npz"))
    T, delay = 6, 2
    pot, stack, boards = z["pot"][:3], z["stack"][:3], z["boards"][:3].astype(np.int64)
    ranges = torch.from_numpy(z["ranges"][:3])
    trees = ptree.build_trees(ptree.root_states(pot, stack, min_raise=2), [0.5, 1.0], int(z["max_depth"]), bb=2,
                              max_raises=int(z["cap"]))
    kw = dict(iterations=T, cfr_type=cfr_type, cfr_plus=cfr_plus, dcfr_delay=delay)
    o = ocfr.SubgameOracle(trees.oracle_dict(boards), ranges, **kw)
    ev = step_evaluator.StepCFREvaluator(trees, boards, ranges, cuda_device, **kw)
    o.initialize()
    ev.initialize_policy_and_beliefs()
    ev.set_leaf_values(0)
    ev.compute_expected_values()
    ev.values_avg.copy_(ev.latest_values)
    _close("start values", ev.latest_values, o.values)
    n = trees.num_roots
    for t in range(T):
        o.iteration(t)
        ev.cfr_iteration(t)
        _close(f"t={t} regrets", ev.cumulative_regrets[n:], o.regrets[n:])
        _close(f"t={t} weight sums", ev.regret_weight_sums[n:], o.weight_sums[n:])
        _close(f"t={t} policy", ev.policy_probs[n:], o.policy[n:])
        _close(f"t={t} policy_avg", ev.policy_probs_avg[n:], o.policy_avg[n:])
        _close(f"t={t} reach", ev.self_reach, o.reach)
        _close(f"t={t} beliefs", ev.beliefs, o.beliefs)
        _close(f"t={t} beliefs_avg", ev.beliefs_avg, o.beliefs_avg)
        _close(f"t={t} values", ev.latest_values, o.values)
    o.finalize()
    ev.update_average_values_final()
    _close("values_avg", ev.values_avg, o.values_avg)
    # the one-call solver ends in the same state
    res, _ = solver.solve_subgames(boards, ranges, pot, stack, iterations=T, max_depth=int(z["max_depth"]),
                                   max_raises=int(z["cap"]), cfr_type=cfr_type, cfr_plus=cfr_plus, dcfr_delay=delay,
                                   device=cuda_device)
    _close("solver policy_avg", res.level_major(res.policy_avg)[n:], ev.policy_probs_avg[n:].cpu())
    _close("solver regrets", res.level_major(res.regrets)[n:], ev.cumulative_regrets[n:].cpu())
    _close("solver root values", res.root_values[..., :1326], ev.values_avg[:n].cpu())


def test_step_methods_with_model_leaves(cuda_device, golden_dir):
    """Turn subgames whose non-fold leaves are valued by a stand-in model, against the upstream run."""
    from poker2_b200 import step_evaluator, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_turn_cap2_t16.npz"))
    trees = ptree.build_trees(ptree.root_states(z["pot"], z["stack"], min_raise=2, street=2), [0.5, 1.0],
                              int(z["max_depth"]), bb=2, max_raises=int(z["cap"]))
    assert trees.total_nodes == int(z["total_nodes"])
    boards = np.concatenate([z["boards"].astype(np.int64), np.full((z["boards"].shape[0], 1), -1)], axis=1)
    w = torch.from_numpy(z["hand_weights"])

    def leaf_fn(beliefs, idx):
        return pot_echo_leaf_fn(trees, idx.cpu(), w)(beliefs)

    ev = step_evaluator.StepCFREvaluator(trees, boards, torch.from_numpy(z["ranges"]), cuda_device,
                                         iterations=int(z["iterations"]), leaf_fn=leaf_fn)
    ev.evaluate_cfr()
    n = trees.num_roots
    _close("policy_probs_avg", ev.policy_probs_avg[n:], z["policy_avg"][n:])
    _close("cumulative_regrets", ev.cumulative_regrets[n:], z["regrets"][n:])
    _close("root values", ev.values_avg[:n], z["root_values"])


def test_graphed_iteration_replays_across_t(cuda_device, golden_dir):
    """`fused_cfr.GraphedCFRIteration` on the step evaluator, the way upstream tests its own
    (tests/test_fused_cfr_triton.py:631-760): capture one `cfr_iteration` at t = 3, restore the state from
    before, then replay it for t = 3, 4, 5 with the device scalars refreshed outside the graph; every replay
    must leave the bits of an uncaptured iteration at that t."""
    from poker2_b200 import fused_cfr as F, step_evaluator, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_batch_cap2_t24.npz"))
    pot, stack, boards = z["pot"][:2], z["stack"][:2], z["boards"][:2].astype(np.int64)
    trees = ptree.build_trees(ptree.root_states(pot, stack, min_raise=2), [0.5, 1.0], int(z["max_depth"]), bb=2,
                              max_raises=int(z["cap"]))

    def fresh():
        ev = step_evaluator.StepCFREvaluator(trees, boards, torch.from_numpy(z["ranges"][:2]), cuda_device, iterations=8)
        ev.initialize_policy_and_beliefs()
        ev.set_leaf_values(0)
        ev.compute_expected_values()
        ev.values_avg.copy_(ev.latest_values)
        for t in range(3):  # past the t = 0 branch of the average-policy update
            ev.cfr_iteration(t)
        return ev

    base, graphed = fresh(), fresh()
    pre = F._EvaluatorStateSnapshot.from_evaluator(graphed)
    runner = F.GraphedCFRIteration(graphed)
    with pytest.raises(RuntimeError):
        runner.replay(3)
    runner.capture(t_capture=3, num_warmup=1)  # the warm-up iterations move the state ...
    assert runner.captured_t == 3
    pre.restore_to(graphed)  # ... so it is put back before the replays
    for t in (3, 4, 5):
        base.cfr_iteration(t)
        runner.replay(t)
        torch.cuda.synchronize()
        diffs = F._EvaluatorStateSnapshot.from_evaluator(base).max_abs_diff(F._EvaluatorStateSnapshot.from_evaluator(graphed))
        print(t, diffs)
        assert max(diffs.values()) == 0.0, (t, diffs)

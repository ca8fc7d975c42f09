"""Subgames with more nodes than the lean iteration kernel holds (160): uncapped river trees of deep stacks
(up to 261 nodes) next to small ones in one batch, and the largest tree the production search settings can
produce (depth 5 over {fold, call, half pot, pot, all-in}: 273 nodes) with leaves valued by a stand-in model.
The one-call solve sends the small subgames through the lean kernel and the large ones through the general
kernel; results must not depend on that."""
import numpy as np
import pytest
import torch

from leaf_models import pot_echo_leaf_fn

pytestmark = pytest.mark.gpu


def _river_batch():
    g = torch.Generator().manual_seed(17)
    stack = np.array([300, 600, 800, 1000, 400, 1000])
    pot = np.full(6, 100)
    boards = torch.stack([torch.randperm(52, generator=g)[:5] for _ in range(6)]).numpy()
    ranges = torch.empty(6, 2, 1326).exponential_(generator=g)
    from oracle import cards

    ranges = ranges * torch.from_numpy(cards.allowed_mask(boards)).float()[:, None, :]
    return boards, ranges / ranges.sum(-1, keepdim=True), pot, stack


def test_mixed_batch_of_small_and_large_river_trees(cuda_device):
    from oracle import cfr as ocfr
    from poker2_b200 import solver, tree as ptree

    boards, ranges, pot, stack = _river_batch()
    T = 7
    trees = ptree.build_trees(ptree.root_states(pot, stack, min_raise=2), [0.5, 1.0], 12, bb=2)
    sizes = np.bincount(trees.root_of)
    assert sizes.tolist() == [89, 173, 233, 261, 121, 261] and int((trees.leaf_mask & ~trees.state.done).sum()) == 0
    o = ocfr.SubgameOracle(trees.oracle_dict(boards), ranges, iterations=T).solve()
    ex, br = o.exploitability()
    N = trees.num_roots
    results = {}
    for name, kw in (("one call", {}), ("general kernel only", dict(lean_iterations=False)), ("device-built trees", dict(device_tree=True))):
        res, _ = solver.solve_subgames(boards, ranges, pot, stack, iterations=T, max_depth=12, max_raises=None,
                                       exploitability=True, device=cuda_device, **kw)
        got = dict(policy_avg=res.level_major(res.policy_avg)[N:].cpu(), regrets=res.level_major(res.regrets)[N:].cpu(),
                   root_values=res.root_values[..., :1326].cpu(), exploitability=res.exploitability.cpu())
        want = dict(policy_avg=o.policy_avg[N:], regrets=o.regrets[N:], root_values=o.values_avg[:N], exploitability=ex)
        for key in got:
            diff = (got[key] - want[key]).abs().max().item()
            print(f"{name} {key}: max abs {diff:.3e}")
            assert torch.equal(got[key], want[key]), (name, key, diff)
        results[name] = got


def test_largest_production_tree_with_model_leaves(cuda_device):
    """Turn roots with deep stacks at depth 5, no raise cap: 273 nodes, 68 of them internal, 144 leaves valued by
    the stand-in model; the pass-by-pass solver against the oracle."""
    from oracle import cfr as ocfr
    from poker2_b200 import solver, tree as ptree

    g = torch.Generator().manual_seed(23)
    n, T = 3, 5
    pot, stack = np.array([20, 300, 30]), np.array([990, 850, 985])
    boards4 = torch.stack([torch.randperm(52, generator=g)[:4] for _ in range(n)]).numpy()
    boards = np.concatenate([boards4, np.full((n, 1), -1)], axis=1)
    ranges = torch.empty(n, 2, 1326).exponential_(generator=g)
    from oracle import cards

    ranges = ranges * torch.from_numpy(cards.allowed_mask(boards4)).float()[:, None, :]
    ranges = ranges / ranges.sum(-1, keepdim=True)
    trees = ptree.build_trees(ptree.root_states(pot, stack, min_raise=10, street=2), [0.5, 1.0], 5, bb=10)
    sizes = np.bincount(trees.root_of)
    assert sizes.max() == 273 and sizes.min() < 160
    w = torch.linspace(-1.0, 1.0, 1326)

    def leaf_fn(beliefs, idx):
        return pot_echo_leaf_fn(trees, idx, w)(beliefs)

    o = ocfr.SubgameOracle(trees.oracle_dict(boards), ranges, iterations=T, leaf_fn=leaf_fn).solve()
    ex, _ = o.exploitability()
    layout = solver.device_layout(trees, boards)
    assert layout.max_internal == 68
    sv = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True)
    fn = pot_echo_leaf_fn(trees, layout.model_nodes, w)
    rb = solver.pad_rows(ranges.to(cuda_device)).contiguous()
    res = sv.solve(rb, solver.iteration_scalars(T), fn)
    assert sv.status() == 0
    for key, got, want in [("policy_avg", res.level_major(res.policy_avg)[n:], o.policy_avg[n:]),
                           ("regrets", res.level_major(res.regrets)[n:], o.regrets[n:]),
                           ("root_values", res.root_values[..., :1326], o.values_avg[:n]), ("exploitability", res.exploitability, ex)]:
        diff = (got.cpu() - want).abs().max().item()
        print(f"{key}: max abs {diff:.3e}")
        torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-6)


def test_evaluator_with_the_production_depth_and_deep_stacks(cuda_device):
    """The evaluator facade on what the production configuration produces early in a hand (stack 1000, blinds
    5 / 10, depth 5, no raise cap, `conf/config_rebel_cfr.yaml:65-73`): flop roots whose trees have 273 nodes,
    leaves valued by a small network averaged over the turn cards."""
    from poker2_b200 import evaluator, leaf_eval, tree as ptree

    g = torch.Generator().manual_seed(4)
    n = 2
    boards = torch.full((n, 5), -1, dtype=torch.int64)
    for i in range(n):
        boards[i, :3] = torch.randperm(52, generator=g)[:3]
    pot, stack = np.array([20, 60]), np.array([990, 970])
    roots = ptree.root_states(pot, stack, min_raise=10, street=1)
    env = evaluator.env_view(roots, boards.numpy())
    model = leaf_eval.ValueMLP(width=64, depth=2, dtype=torch.float32, seed=2).to(cuda_device)
    ev = evaluator.SubgameEvaluator(cuda_device, iterations=3, max_depth=5, bb=10, max_raises=None, model=model,
                                    leaf_chunk=64, generator=torch.Generator().manual_seed(1))
    ranges = torch.empty(n, 2, 1326).exponential_(generator=g)
    hit = torch.zeros(n, 52, dtype=torch.bool)
    hit.scatter_(1, boards[:, :3], True)
    c1, c2 = np.triu_indices(52, k=1)
    ranges = ranges * (~(hit[:, torch.from_numpy(c1)] | hit[:, torch.from_numpy(c2)]))[:, None, :]
    ranges = ranges / ranges.sum(-1, keepdim=True)
    ev.initialize_subgame(env, torch.arange(n), ranges)
    assert np.bincount(ev.trees.root_of).max() == 273 and ev.layout.num_model_leaves > 0
    ev.evaluate_cfr()
    value_batch, pre_batch, policy_batch = ev.training_data()
    assert len(value_batch) == n
    for t in (value_batch.value_targets, policy_batch.policy_targets):
        assert torch.isfinite(t).all()
    assert np.isfinite(ev.stats["local_exploitability"]) and ev.stats["evaluator_total_nodes"] == float(ev.trees.total_nodes)
    # the policy targets are distributions over the legal actions
    sums = policy_batch.policy_targets.sum(dim=-1)
    torch.testing.assert_close(sums, torch.ones_like(sums), rtol=1e-4, atol=1e-4)


DEFAULT_BINS = [0.5, 0.75, 1.0, 1.5, 2.0]  # EnvConfig.bet_bins of the upstream dataclass: 8 actions per node


def test_eight_actions_per_node_on_terminal_trees(cuda_device):
    """River subgames over the dataclass-default bet sizes (fold, call, five bets, all-in) with a raise cap, so
    that every leaf is terminal: nodes with 6, 7 and 8 children, trees of 59 ... 207 nodes in one batch.  The
    one-call solve keeps such a batch in the general kernel (its wide build); equal bits with the oracle."""
    from oracle import cards, cfr as ocfr
    from poker2_b200 import solver, tree as ptree

    g = torch.Generator().manual_seed(29)
    pot, stack = np.array([100, 40, 200, 100]), np.array([400, 1000, 300, 250])
    n, T = 4, 6
    boards = torch.stack([torch.randperm(52, generator=g)[:5] for _ in range(n)]).numpy()
    ranges = torch.empty(n, 2, 1326).exponential_(generator=g) * torch.from_numpy(cards.allowed_mask(boards)).float()[:, None, :]
    ranges = ranges / ranges.sum(-1, keepdim=True)
    trees = ptree.build_trees(ptree.root_states(pot, stack, min_raise=2), DEFAULT_BINS, 12, bb=2, max_raises=2)
    assert np.bincount(trees.root_of).tolist() == [159, 207, 59, 117] and int(trees.child_count.max()) == 8
    o = ocfr.SubgameOracle(trees.oracle_dict(boards), ranges, iterations=T).solve()
    ex, _ = o.exploitability()
    for kw in ({}, dict(device_tree=True)):
        res, _ = solver.solve_subgames(boards, ranges, pot, stack, iterations=T, bet_bins=DEFAULT_BINS, max_depth=12,
                                       max_raises=2, exploitability=True, device=cuda_device, **kw)
        for key, got, want in [("policy_avg", res.level_major(res.policy_avg)[n:], o.policy_avg[n:]),
                               ("regrets", res.level_major(res.regrets)[n:], o.regrets[n:]),
                               ("root_values", res.root_values[..., :1326], o.values_avg[:n]), ("exploitability", res.exploitability, ex)]:
            diff = (got.cpu() - want).abs().max().item()
            print(f"{kw} {key}: max abs {diff:.3e}")
            assert torch.equal(got.cpu(), want), (key, diff)


def test_default_bet_sizes_at_depth_three_with_model_leaves(cuda_device):
    """The dataclass-default bet sizes without a raise cap at depth 3: up to 282 nodes, 8 children, most leaves
    valued by the stand-in model; pass-by-pass solver against the oracle."""
    from oracle import cards, cfr as ocfr
    from poker2_b200 import solver, tree as ptree

    g = torch.Generator().manual_seed(31)
    pot, stack = np.array([20, 100, 200]), np.array([990, 400, 300])
    n, T = 3, 5
    boards = torch.stack([torch.randperm(52, generator=g)[:5] for _ in range(n)]).numpy()
    ranges = torch.empty(n, 2, 1326).exponential_(generator=g) * torch.from_numpy(cards.allowed_mask(boards)).float()[:, None, :]
    ranges = ranges / ranges.sum(-1, keepdim=True)
    trees = ptree.build_trees(ptree.root_states(pot, stack, min_raise=2), DEFAULT_BINS, 3, bb=2)
    assert np.bincount(trees.root_of).tolist() == [282, 143, 52] and int(trees.child_count.max()) == 8
    w = torch.linspace(-1.0, 1.0, 1326)
    o = ocfr.SubgameOracle(trees.oracle_dict(boards), ranges, iterations=T,
                           leaf_fn=lambda b, idx: pot_echo_leaf_fn(trees, idx, w)(b)).solve()
    ex, _ = o.exploitability()
    layout = solver.device_layout(trees, boards)
    sv = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True)
    res = sv.solve(solver.pad_rows(ranges.to(cuda_device)).contiguous(), solver.iteration_scalars(T),
                   pot_echo_leaf_fn(trees, layout.model_nodes, w))
    assert sv.status() == 0
    for key, got, want in [("policy_avg", res.level_major(res.policy_avg)[n:], o.policy_avg[n:]),
                           ("regrets", res.level_major(res.regrets)[n:], o.regrets[n:]),
                           ("root_values", res.root_values[..., :1326], o.values_avg[:n]), ("exploitability", res.exploitability, ex)]:
        diff = (got.cpu() - want).abs().max().item()
        print(f"{key}: max abs {diff:.3e}")
        torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("warm", [False, True])
def test_joint_sweeps_equal_separate_launches(cuda_device, warm):
    """A pass as one launch (bottom-up sweep of the pass before it + its own top-down sweep, `phases` 16) against
    the two launches per pass: same bits, on trees of 52 ... 282 nodes with model leaves, with and without a
    warm start (whose seeding keeps the first two sweeps apart)."""
    from oracle import cards
    from poker2_b200 import solver, tree as ptree

    g = torch.Generator().manual_seed(37)
    pot, stack = np.array([20, 100, 200, 60]), np.array([990, 400, 300, 970])
    n, T = 4, 6
    boards = torch.stack([torch.randperm(52, generator=g)[:5] for _ in range(n)]).numpy()
    ranges = torch.empty(n, 2, 1326).exponential_(generator=g) * torch.from_numpy(cards.allowed_mask(boards)).float()[:, None, :]
    ranges = ranges / ranges.sum(-1, keepdim=True)
    trees = ptree.build_trees(ptree.root_states(pot, stack, min_raise=2), DEFAULT_BINS, 3, bb=2)
    layout = solver.device_layout(trees, boards)
    w = torch.linspace(-1.0, 1.0, 1326)
    fn = pot_echo_leaf_fn(trees, layout.model_nodes, w)
    rb = solver.pad_rows(ranges.to(cuda_device)).contiguous()
    scal = solver.iteration_scalars(T, warm_start_iterations=2 if warm else 0)
    kw = {}
    if warm:
        cc = torch.from_numpy(trees.child_count[trees.parent_index.clip(min=0)]).clamp(min=1)
        kw = dict(start_policy=(1.0 / cc.float())[:, None].expand(-1, 1326).contiguous(), warm_start_iterations=2,
                  warm_start_multiplier=3.0)
    out, launches = [], []
    for joint in (False, True):
        sv = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True, sampling=True)
        sv.set_sampling_schedule(torch.tensor([2, 3, 5, 4]), warm_start_iterations=2 if warm else 0)
        res = sv.solve(rb, scal, fn, joint_sweeps=joint, **kw)
        assert sv.status() == 0
        launches.append(sv.launches)
        out.append([x.clone() for x in (res.policy_avg, res.regrets, res.weight_sums, res.root_values, res.exploitability,
                                        res.policy_sample, res.beliefs_last)])
    assert launches[1] < launches[0]
    for a, b in zip(*out):
        assert torch.equal(a, b)


def test_production_tree_shape_against_the_upstream_run(cuda_device, golden_dir):
    """The same trees (depth 5, no raise cap, 273 and 242 nodes) solved pass by pass on the GPU, against the
    arrays the upstream evaluator produced."""
    import os

    from poker2_b200 import solver, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_depth5_nocap_t6.npz"))
    trees = ptree.build_trees(ptree.root_states(z["pot"], z["stack"], min_raise=2, street=2), [0.5, 1.0],
                              int(z["max_depth"]), bb=2)
    assert trees.total_nodes == int(z["total_nodes"])
    boards = np.concatenate([z["boards"].astype(np.int64), np.full((2, 1), -1)], axis=1)
    layout = solver.device_layout(trees, boards)
    sv = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True)
    fn = pot_echo_leaf_fn(trees, layout.model_nodes, torch.from_numpy(z["hand_weights"]))
    rb = solver.pad_rows(torch.from_numpy(z["ranges"]).to(cuda_device)).contiguous()
    res = sv.solve(rb, solver.iteration_scalars(int(z["iterations"])), fn)
    assert sv.status() == 0
    rows = torch.from_numpy(z["rows"])
    for key, got, want in [("policy_avg", res.level_major(res.policy_avg).cpu()[rows], z["policy_avg_rows"]),
                           ("regrets", res.level_major(res.regrets).cpu()[rows], z["regrets_rows"]),
                           ("root_values", res.root_values[..., :1326].cpu(), z["root_values"]),
                           ("exploitability", res.exploitability.cpu(), z["exploitability"]),
                           ("br_values", res.br_values.cpu(), z["br_values"])]:
        want = torch.from_numpy(want)
        print(f"{key}: max abs {(got - want).abs().max().item():.3e}")
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)


def test_default_bet_sizes_against_the_upstream_run(cuda_device, golden_dir):
    """Eight actions per node at depth 3 (280 and 143 nodes, model leaves at the depth limit) on the GPU, against
    the arrays of the upstream run."""
    import os

    from poker2_b200 import solver, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_default_bins_depth3_t6.npz"))
    bins = [float(x) for x in z["bet_bins"]]
    trees = ptree.build_trees(ptree.root_states(z["pot"], z["stack"], min_raise=2), bins, int(z["max_depth"]), bb=2)
    assert trees.total_nodes == int(z["total_nodes"])
    boards = z["boards"].astype(np.int64)
    layout = solver.device_layout(trees, boards)
    assert layout.max_children == 8
    sv = solver.SteppedSolver(layout, torch.from_numpy(boards), cuda_device, exploitability=True)
    fn = pot_echo_leaf_fn(trees, layout.model_nodes, torch.from_numpy(z["hand_weights"]))
    rb = solver.pad_rows(torch.from_numpy(z["ranges"]).to(cuda_device)).contiguous()
    res = sv.solve(rb, solver.iteration_scalars(int(z["iterations"])), fn)
    assert sv.status() == 0
    rows = torch.from_numpy(z["rows"])
    for key, got, want in [("policy_avg", res.level_major(res.policy_avg).cpu()[rows], z["policy_avg_rows"]),
                           ("regrets", res.level_major(res.regrets).cpu()[rows], z["regrets_rows"]),
                           ("root_values", res.root_values[..., :1326].cpu(), z["root_values"]),
                           ("exploitability", res.exploitability.cpu(), z["exploitability"]),
                           ("br_values", res.br_values.cpu(), z["br_values"])]:
        want = torch.from_numpy(want)
        print(f"{key}: max abs {(got - want).abs().max().item():.3e}")
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)

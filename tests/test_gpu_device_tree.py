"""Trees expanded on the GPU (`p2b_tree_count` / `p2b_tree_records`) against the host builder,
which is itself pinned to the upstream environment (tests/test_tree_and_oracle_cfr.py): the
node and subgame records must be byte-identical, and so must every derived index array."""
import numpy as np
import pytest
import torch

from poker2_b200 import device_tree, leaf_eval, solver
from poker2_b200 import tree as ptree

pytestmark = pytest.mark.gpu


def random_roots(rng, n, street, *, short=False, general=False):
    pot = rng.integers(2, 60 if short else 400, size=n)
    stacks = rng.integers(0 if short else 50, 80 if short else 1200, size=(n, 2))
    roots = ptree.root_states(pot, stacks, street=street, button=rng.integers(0, 2, size=n))
    if general:  # roots in the middle of a betting round
        roots.committed[:, 0] = rng.integers(0, 30, size=n)
        roots.committed[:, 1] = rng.integers(0, 30, size=n)
        roots.actions_this_round[:] = rng.integers(0, 3, size=n)
        roots.to_act[:] = rng.integers(0, 2, size=n)
        roots.min_raise[:] = rng.integers(2, 20, size=n)
        roots.raises[:] = rng.integers(0, 2, size=n)
        roots.is_allin[:, 0] = stacks[:, 0] == 0
        roots.is_allin[:, 1] = stacks[:, 1] == 0
    return roots


def random_boards(rng, n, cards):
    out = np.full((n, 5), -1, dtype=np.int64)
    for i in range(n):
        out[i, :cards] = rng.choice(52, size=cards, replace=False)
    return out


CASES = [
    # street, board cards, bet bins, max_depth, max_raises, short stacks, general roots
    (3, 5, [0.5, 1.0], 8, 2, False, False),
    (3, 5, [0.5, 1.0], 4, None, False, False),
    (3, 5, [0.5, 1.0], 8, 3, True, False),
    (2, 4, [0.5, 1.0], 8, 2, False, False),
    (1, 3, [0.75], 5, None, False, False),
    (3, 5, [], 8, None, True, False),
    (3, 5, [0.33, 0.66, 1.0], 2, None, False, False),
    (2, 4, [0.5, 1.0], 8, 2, True, True),
    (3, 5, [1.0], 2, None, False, True),
]


@pytest.mark.parametrize("case", range(len(CASES)))
def test_device_tree_equals_host_tree(cuda_device, case):
    street, cards, bins, depth, cap, short, general = CASES[case]
    rng = np.random.default_rng(100 + case)
    n = 257
    roots = random_roots(rng, n, street, short=short, general=general)
    boards = random_boards(rng, n, cards)
    bb = rng.integers(1, 5, size=n) if general else 2
    trees = ptree.build_trees(roots, bins, depth, bb=bb, max_raises=cap)
    want = solver.device_layout(trees, boards)
    got = device_tree.build_device_layout(roots, boards, bins, depth, bb=bb, max_raises=cap, device=cuda_device,
                                          node_state=True)
    assert got.rows == want.rows
    assert got.nodes.tobytes() == want.nodes.tobytes()
    assert got.subgames.tobytes() == want.subgames.tobytes()
    assert np.array_equal(got.to_level_major, want.to_level_major)
    assert np.array_equal(got.from_level_major, want.from_level_major)
    assert np.array_equal(got.leaf_begin, want.leaf_begin)
    assert np.array_equal(got.model_rows, want.model_rows)
    assert np.array_equal(got.model_nodes, want.model_nodes)
    assert (got.max_internal, got.max_children, got.tree_depth) == (want.max_internal, want.max_children, want.tree_depth)
    assert got.depth_offsets == [int(x) for x in trees.depth_offsets]
    assert np.array_equal(got.root_of_row_dev.cpu().numpy(), trees.root_of[want.to_level_major])
    st = got.node_state_dev.cpu().numpy()
    lm = want.to_level_major
    assert np.array_equal(st[:, 0], trees.state.pot[lm]) and np.array_equal(st[:, 1:3], trees.state.stacks[lm])
    assert np.array_equal(st[:, 5], trees.state.street[lm]) and np.array_equal(st[:, 6], trees.state.to_act[lm])
    if got.num_model_leaves:
        ctx = leaf_eval.leaf_context(trees, want.model_nodes)
        assert torch.equal(got.leaf_context().cpu(), ctx)


def test_device_tree_reports_oversized_subgames(cuda_device):
    roots = ptree.root_states(np.array([100, 100]), np.array([20000, 400]))
    boards = random_boards(np.random.default_rng(0), 2, 5)
    with pytest.raises(ValueError, match="more than 320 nodes"):
        device_tree.build_device_layout(roots, boards, [0.25, 0.5, 1.0], 12, device=cuda_device)


def test_device_tree_reports_too_many_actions(cuda_device):
    roots = ptree.root_states(np.array([100]), np.array([5000]))
    boards = random_boards(np.random.default_rng(0), 1, 5)
    with pytest.raises(ValueError, match="actions per node"):
        device_tree.build_device_layout(roots, boards, [0.2, 0.3, 0.4, 0.5, 0.75, 1.0, 1.5], 1, device=cuda_device)


def test_solve_on_device_tree_equals_solve_on_host_tree(cuda_device):
    import bench

    boards, ranges, pot, stack = bench.make_inputs(24, 5)
    kw = dict(iterations=12, max_raises=2, device=cuda_device, exploitability=True)
    a, trees = solver.solve_subgames(boards, ranges, pot, stack, **kw)
    b, none = solver.solve_subgames(boards, ranges, pot, stack, device_tree=True, **kw)
    assert none is None and trees is not None
    torch.cuda.synchronize()
    for name in ("policy_avg", "regrets", "root_values", "exploitability"):
        assert torch.equal(getattr(a, name), getattr(b, name)), name
    assert torch.equal(a.level_major(a.policy_avg), b.level_major(b.policy_avg))


def test_network_leaves_on_device_tree_equal_host_tree(cuda_device):
    from poker2_b200 import leaf_eval

    rng = np.random.default_rng(5)
    n, iterations = 6, 5
    boards = torch.from_numpy(random_boards(rng, n, 4)[:, :4].copy())
    ranges = torch.rand(n, 2, 1326, generator=torch.Generator().manual_seed(5))
    for i in range(n):  # zero the blocked combos, normalise
        ok = torch.from_numpy(~np.isin(np.array(np.triu_indices(52, 1)).T, boards[i].numpy()).any(axis=1))
        ranges[i] *= ok
    ranges /= ranges.sum(dim=-1, keepdim=True)
    pot = torch.from_numpy(rng.integers(20, 200, size=n))
    stack = torch.from_numpy(rng.integers(100, 1000, size=n))
    out = []
    for dev_tree in (False, True):
        model = leaf_eval.ValueMLP(width=64, depth=2, dtype=torch.float32, seed=3).to(cuda_device)
        res, trees, sv = solver.solve_subgames_with_model(
            boards, ranges, pot, stack, model, street=2, iterations=iterations, max_raises=2, device=cuda_device,
            chunk=16, device_tree=dev_tree)
        assert sv.layout.num_model_leaves > 0
        out.append((res.policy_avg.clone(), res.root_values.clone(), res.regrets.clone()))
    for a, b in zip(*out):
        assert torch.equal(a, b)

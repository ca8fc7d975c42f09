"""The default choice of the kernel for the iteration passes of a one-call solve: small batches go to the general
kernel, the others to the lean kernel (with the general kernel taking the subgames that are too large for it).
The iteration-kernel timer tells which one ran; the results must be the same bits under both policies."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _lean_ran(fn):
    """Runs fn with the iteration-kernel timer on; True if the lean kernel was launched."""
    from poker2_b200 import _lib

    _lib.call("p2b_cfr_iteration_timing", 1)
    try:
        fn()
        torch.cuda.synchronize()
        ms = ctypes.c_float(0.0)
        rc = _lib.lib().p2b_cfr_iteration_ms(ctypes.byref(ms))
        return rc == 0
    finally:
        _lib.call("p2b_cfr_iteration_timing", 0)


@pytest.fixture
def auto_policy():
    from poker2_b200 import solver

    before = solver.set_path_policy("auto")
    yield
    solver.set_path_policy(before)


def test_default_policy_by_batch_size(cuda_device, auto_policy):
    import bench
    from poker2_b200 import solver, tree as ptree

    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    results = {}
    for B in (sms, sms + 1):
        boards, ranges, pot, stack = bench.make_inputs(B, 2)
        trees = ptree.build_trees(ptree.root_states(pot.numpy(), stack.numpy()), [0.5, 1.0], 8, max_raises=2)
        layout = solver.device_layout(trees, boards.numpy())
        rb = solver.pad_rows(ranges.to(cuda_device)).contiguous()
        scal = solver.iteration_scalars(4)
        sv = solver.SubgameSolver(layout, boards, cuda_device, exploitability=True)
        lean = _lean_ran(lambda: sv.solve(rb, scal))
        assert lean == (B > sms), (B, lean)  # one subgame per SM or fewer: the general kernel
        got = [x.clone() for x in (sv.policy_avg, sv.regrets, sv.root_values, sv.exploitability)]
        solver.set_path_policy("lean")
        try:
            sv2 = solver.SubgameSolver(layout, boards, cuda_device, exploitability=True)
            assert _lean_ran(lambda: sv2.solve(rb, scal))
            for a, b in zip(got, (sv2.policy_avg, sv2.regrets, sv2.root_values, sv2.exploitability)):
                assert torch.equal(a, b)
        finally:
            solver.set_path_policy("auto")
        results[B] = lean


def test_default_policy_with_large_subgames(cuda_device, auto_policy):
    """A small batch in which some subgame exceeds the lean kernel's node limit stays in the general kernel."""
    from poker2_b200 import solver, tree as ptree

    g = torch.Generator().manual_seed(3)
    B = 200
    pot = np.full(B, 100)
    stack = np.where(np.arange(B) % 5 == 0, 1000, 300)
    boards = torch.stack([torch.randperm(52, generator=g)[:5] for _ in range(B)])
    ranges = torch.empty(B, 2, 1326).exponential_(generator=g)
    ranges = ranges / ranges.sum(-1, keepdim=True)
    trees = ptree.build_trees(ptree.root_states(pot, stack, min_raise=2), [0.5, 1.0], 12, bb=2)
    assert np.bincount(trees.root_of).max() > 160
    layout = solver.device_layout(trees, boards.numpy())
    rb = solver.pad_rows(ranges.to(cuda_device)).contiguous()
    scal = solver.iteration_scalars(3)
    sv = solver.SubgameSolver(layout, boards, cuda_device)
    assert not _lean_ran(lambda: sv.solve(rb, scal))
    got = [x.clone() for x in (sv.policy_avg, sv.regrets, sv.root_values)]
    solver.set_path_policy("lean")
    sv2 = solver.SubgameSolver(layout, boards, cuda_device)
    assert _lean_ran(lambda: sv2.solve(rb, scal))
    for a, b in zip(got, (sv2.policy_avg, sv2.regrets, sv2.root_values)):
        assert torch.equal(a, b)

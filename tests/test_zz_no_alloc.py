"""The allocation-free solve entry point (`p2b_cfr_solve_noalloc`) against the regular one.

Some hosts of the library cannot allocate GPU memory when they call it: a data-generation
worker confined to a memory slice its trainer handed out, a caller in a latency-critical
loop (a driver allocation stalls the device), a process whose framework pool already owns
all free memory.  For them the library carries a fixed 32 MiB work area; this test checks
that solving through it gives what the regular entry point gives, twice in a row with a
different batch solved through the area in between (the area keeps the previous call's
contents, so the second comparison proves nothing stale leaks in), that free device memory
does not move across a call, and that a refused batch is reported by the status call.
The file name sorts last on purpose: a run that stops at the first failure has then
already executed every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-6  # same tolerance as the other CFR tests; in practice the match is exact


def _inputs(n, seed):
    g = torch.Generator().manual_seed(seed)
    boards = torch.stack([torch.randperm(52, generator=g)[:5] for _ in range(n)])
    hit = torch.zeros(n, 52, dtype=torch.bool).scatter_(1, boards, True)
    c1, c2 = np.triu_indices(52, k=1)
    blocked = hit[:, torch.from_numpy(c1)] | hit[:, torch.from_numpy(c2)]
    ranges = torch.empty(n, 2, 1326).exponential_(generator=g) * (~blocked)[:, None, :]
    ranges = ranges / ranges.sum(-1, keepdim=True)
    pot = torch.randint(20, 201, (n,), generator=g)
    stack = torch.randint(100, 1001, (n,), generator=g)
    return boards, ranges, pot, stack


def test_noalloc_entry_matches_regular_entry(cuda_device):
    from poker2_b200 import _lib, solver
    from poker2_b200 import tree as ptree

    n, iterations = 80, 12  # more subgames than the fixed area has room for blocks at once
    boards, ranges, pot, stack = _inputs(n, seed=31)
    trees = ptree.build_trees(ptree.root_states(pot.numpy(), stack.numpy()), [0.5, 1.0], 8, max_raises=2)
    layout = solver.device_layout(trees, boards.numpy())
    scal = solver.iteration_scalars(iterations)
    rb = solver.pad_rows(ranges.to(cuda_device)).contiguous()

    ref_solver = solver.SubgameSolver(layout, boards, cuda_device, keep_policy=True)
    ref = ref_solver.solve(rb, scal)
    want = {k: getattr(ref, k).clone() for k in ("policy_avg", "regrets", "weight_sums", "policy", "root_values")}

    sv = solver.SubgameSolver(layout, boards, cuda_device, keep_policy=True)
    scal_dev = torch.from_numpy(scal.view(np.uint8).reshape(iterations, 32).copy()).to(cuda_device)
    assert _lib.lib().p2b_cfr_noalloc_scratch_floats() * 4 == 32 << 20
    # another batch (other boards, pots, stacks: other trees) that dirties the shared area between the calls
    boards2, ranges2, pot2, stack2 = _inputs(n, seed=77)
    trees2 = ptree.build_trees(ptree.root_states(pot2.numpy(), stack2.numpy()), [0.5, 1.0], 8, max_raises=2)
    other = solver.SubgameSolver(solver.device_layout(trees2, boards2.numpy()), boards2, cuda_device)
    rb2 = solver.pad_rows(ranges2.to(cuda_device)).contiguous()
    for call in range(2):
        for buf in (sv.policy_avg, sv.regrets, sv.weight_sums, sv.policy, sv.root_values):
            buf.fill_(float("nan"))  # whatever the previous call left must be overwritten
        if call == 1:
            solver.solve_noalloc(other, rb2, scal_dev)
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info(cuda_device)[0]
        got = solver.solve_noalloc(sv, rb, scal_dev)
        torch.cuda.synchronize()
        if call == 1:  # the first call on a device sets the area up; later calls must not move free memory
            assert torch.cuda.mem_get_info(cuda_device)[0] == free_before
        assert solver.noalloc_status(cuda_device) == 0
        for k, w in want.items():
            g = getattr(got, k)
            rows = slice(None) if g.dim() == 3 else torch.from_numpy(layout.from_level_major[n:]).to(cuda_device)
            torch.testing.assert_close(g[rows][..., :1326], w[rows][..., :1326], rtol=RTOL, atol=ATOL,
                                       msg=lambda m, k=k, call=call: f"{k} (call {call}): {m}")


def test_noalloc_entry_rejects_oversized_trees(cuda_device):
    from poker2_b200 import _lib, solver
    from poker2_b200 import tree as ptree

    boards, ranges, pot, stack = _inputs(1, seed=5)
    trees = ptree.build_trees(ptree.root_states(pot.numpy(), stack.numpy()), [0.5, 1.0], 8, max_raises=2)
    layout = solver.device_layout(trees, boards.numpy())
    sv = solver.SubgameSolver(layout, boards, cuda_device)
    per_block = 6 * 1344
    layout.max_internal = int(_lib.lib().p2b_cfr_noalloc_scratch_floats()) // per_block + 1  # one too many
    scal = solver.iteration_scalars(2)
    scal_dev = torch.from_numpy(scal.view(np.uint8).reshape(2, 32).copy()).to(cuda_device)
    rb = solver.pad_rows(ranges.to(cuda_device)).contiguous()
    with pytest.raises(RuntimeError, match="built-in work area"):
        solver.solve_noalloc(sv, rb, scal_dev)


def test_noalloc_entry_reports_a_refused_batch(cuda_device):
    """A malformed record makes the call solve nothing; the status call says which subgame."""
    from poker2_b200 import solver
    from poker2_b200 import tree as ptree

    n = 6
    boards, ranges, pot, stack = _inputs(n, seed=9)
    trees = ptree.build_trees(ptree.root_states(pot.numpy(), stack.numpy()), [0.5, 1.0], 8, max_raises=2)
    layout = solver.device_layout(trees, boards.numpy())
    victim = 4
    layout.nodes[int(layout.subgames[victim]["node_begin"])]["first_child"] = 0  # the root as its own child
    sv = solver.SubgameSolver(layout, boards, cuda_device)
    scal = solver.iteration_scalars(3)
    scal_dev = torch.from_numpy(scal.view(np.uint8).reshape(3, 32).copy()).to(cuda_device)
    rb = solver.pad_rows(ranges.to(cuda_device)).contiguous()
    sv.root_values.fill_(-7.0)
    got = solver.solve_noalloc(sv, rb, scal_dev)
    assert solver.noalloc_status(cuda_device) == victim + 1
    assert bool((got.root_values == -7.0).all())

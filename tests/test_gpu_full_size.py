"""The benchmark configurations at their full sizes, checked through properties that do not
need the oracle on every element: independence of the subgames of a batch, agreement with the
oracle on a subsample, exact category frequencies, value cancellation."""
import numpy as np
import pytest
import torch

from oracle import cards, rank7

pytestmark = pytest.mark.gpu


def test_river_batch_4096_subgames(cuda_device):
    """B = 4096 river subgames (few iterations): every subgame is solved as if alone, the
    average policy is a distribution over the children, and two subgames match the oracle."""
    import bench
    from oracle import cfr as ocfr
    from poker2_b200 import solver, tree as ptree

    B, T = 4096, 6
    boards, ranges, pot, stack = bench.make_inputs(B, 2)
    res, trees = solver.solve_subgames(boards, ranges, pot, stack, iterations=T, max_raises=2, device=cuda_device,
                                       exploitability=True)
    layout = res.layout
    assert torch.isfinite(res.exploitability).all() and (res.exploitability > -1e-4).all()
    # (a) a slice of the batch solved on its own gives the same bits
    pick = np.r_[0:6, B - 6:B]
    sub, sub_trees = solver.solve_subgames(boards[pick], ranges[pick], pot[pick], stack[pick], iterations=T,
                                           max_raises=2, device=cuda_device, exploitability=True)
    for s_local, s_global in enumerate(pick):
        a = layout.subgames[s_global]
        b = sub.layout.subgames[s_local]
        assert a["n_nodes"] == b["n_nodes"]
        ra = slice(int(a["node_begin"]), int(a["node_begin"] + a["n_nodes"]))
        rb = slice(int(b["node_begin"]), int(b["node_begin"] + b["n_nodes"]))
        assert torch.equal(res.regrets[ra], sub.regrets[rb])
        assert torch.equal(res.policy_avg[ra], sub.policy_avg[rb])
        assert torch.equal(res.root_values[s_global], sub.root_values[s_local])
        assert torch.equal(res.exploitability[s_global], sub.exploitability[s_local])
    # (b) the average policy sums to one over the children of every internal node, per allowed hand
    pol = res.level_major(res.policy_avg).cpu()
    N, top = trees.num_roots, trees.depth_offsets[-2]
    sums = torch.zeros(top, 1326)
    sums.index_add_(0, torch.from_numpy(trees.parent_index[N:]), pol[N:])
    internal = torch.from_numpy(trees.child_count[:top] > 0)
    allowed = torch.from_numpy(cards.allowed_mask(boards.numpy()))[torch.from_numpy(trees.root_of[:top])]
    dev = (sums - 1.0).abs()[internal][allowed[internal]]
    assert dev.max().item() < 1e-5
    # (c) every 64th subgame of the batch (64 roots, ragged trees) against the oracle: the rows the full
    # batch produced for them, not a separate solve
    pick = np.arange(0, B, 64)
    t2 = ptree.build_trees(ptree.root_states(pot[pick].numpy(), stack[pick].numpy()), [0.5, 1.0], 8, max_raises=2)
    o = ocfr.SubgameOracle(t2.oracle_dict(boards[pick].numpy()), ranges[pick], iterations=T).solve()
    ex, _ = o.exploitability()
    sub_layout = solver.device_layout(t2, boards[pick].numpy())
    to_level = torch.from_numpy(np.asarray(sub_layout.from_level_major))  # level-major row -> subgame-major row of the subsample
    rows = []
    for s_local, s_global in enumerate(pick):
        a, b = layout.subgames[s_global], sub_layout.subgames[s_local]
        assert a["n_nodes"] == b["n_nodes"]
        rows.append(torch.arange(int(a["node_begin"]), int(a["node_begin"] + a["n_nodes"])))
    rows = torch.cat(rows).to(cuda_device)  # rows of the full batch in the subsample's subgame-major order
    pol = res.policy_avg[rows][to_level.to(cuda_device)][:, :1326].cpu()
    reg = res.regrets[rows][to_level.to(cuda_device)][:, :1326].cpu()
    n2 = len(pick)
    torch.testing.assert_close(pol[n2:], o.policy_avg[n2:], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(reg[n2:], o.regrets[n2:], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(res.root_values[torch.from_numpy(pick).to(cuda_device)][..., :1326].cpu(), o.values_avg[:n2],
                               rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(res.exploitability[torch.from_numpy(pick).to(cuda_device)].cpu(), ex, rtol=1e-4, atol=1e-6)


def test_rank_2_pow_26_hands(cuda_device):
    """2^26 random seven-card hands: a strided subsample equals the oracle, and the hand-type
    histogram matches the exact frequencies over all C(52,7) hands within sampling error."""
    from poker2_b200 import rules

    n = 1 << 26
    g = torch.Generator(device=cuda_device).manual_seed(1)
    chunks = [torch.rand((n // 16, 52), device=cuda_device, generator=g).argsort(dim=1)[:, :7].to(torch.int16)
              for _ in range(16)]
    hands = torch.cat(chunks)
    del chunks
    got = rules.rank_7_cards_single_batch(hands)
    assert got.shape == (n,) and got.dtype == torch.int32
    stride = 64
    sample = hands[::stride].cpu().numpy()
    assert np.array_equal(got[::stride].cpu().numpy(), rank7.rank7(sample, rank7.MODE_IDS))
    types = torch.bincount((got >> 20).to(torch.int64), minlength=10).cpu().numpy().astype(np.float64)
    exact = {9: 41584, 8: 224848, 7: 3473184, 6: 4047644, 5: 6180020, 4: 6461620, 3: 31433400, 2: 58627800,
             1: 23294460}
    total = float(sum(exact.values()))
    assert total == 133784560.0 and types[0] == 0
    for t, cnt in exact.items():
        p = cnt / total
        sigma = np.sqrt(n * p * (1 - p))
        assert abs(types[t] - n * p) < 6 * sigma, (t, types[t], n * p)


def test_showdown_4096_boards(cuda_device):
    """4096 river boards with two Dirichlet(1) ranges each: 24 of them equal the oracle, and on
    all of them what one player wins the other loses."""
    import bench
    from oracle import showdown as oshow, unblocked
    from poker2_b200 import showdown

    m = 4096
    boards, ranges, _, _ = bench.make_inputs(m, 1)
    tabs = showdown.BoardTables(boards.to(cuda_device))
    ones = torch.ones(m, 2, dtype=torch.int64)
    vals = showdown.showdown_values(tabs, ranges.to(cuda_device).contiguous(), ones, torch.ones(m)).cpu()
    pick = torch.arange(0, m, m // 24)[:24]
    want = oshow.showdown_values(boards[pick].numpy(), ranges[pick], ones[pick], torch.ones(len(pick)))
    torch.testing.assert_close(vals[pick], want, rtol=1e-5, atol=1e-6)
    w0 = ranges[:, 0].double() * unblocked.unblocked_mass(ranges[:, 1]).double()
    w1 = ranges[:, 1].double() * unblocked.unblocked_mass(ranges[:, 0]).double()
    total = (vals[:, 0].double() * w0).sum(-1) + (vals[:, 1].double() * w1).sum(-1)
    assert total.abs().max().item() < 1e-5

"""CUDA showdown evaluation (through the C ABI) against the oracle and golden values."""
import os

import numpy as np
import pytest
import torch

from oracle import cards
from oracle import showdown as oshow

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-6  # fp32 values; tolerance stated by the project brief (1e-5 relative)


def test_showdown_golden(cuda_device, golden_dir):
    from poker2_b200 import showdown

    z = np.load(os.path.join(golden_dir, "showdown.npz"))
    tabs = showdown.BoardTables(torch.from_numpy(z["boards"]).to(cuda_device))
    got = showdown.showdown_values(tabs, torch.from_numpy(z["beliefs"]).to(cuda_device),
                                   torch.from_numpy(z["potential"]), torch.from_numpy(z["scale"]))
    want = torch.from_numpy(z["values"])
    torch.testing.assert_close(got.cpu(), want, rtol=RTOL, atol=ATOL)
    # the stated bar is the tolerance above; what the kernel delivers is every bit of upstream's fp32 values
    assert torch.equal(got.cpu(), want), int((got.cpu() != want).sum())


def test_showdown_random_boards_shared_tables(cuda_device):
    from poker2_b200 import showdown

    g = torch.Generator().manual_seed(3)
    nb, rows = 5, 23
    boards = torch.stack([torch.randperm(52, generator=g)[:5] for _ in range(nb)])
    table_of_row = torch.randint(0, nb, (rows,), generator=g)
    allowed = torch.from_numpy(cards.allowed_mask(boards.numpy()))[table_of_row]
    bel = torch.empty(rows, 2, 1326).exponential_(generator=g) * allowed[:, None].float()
    bel[0, 0] = 0  # an empty range: every denominator hits the clamp
    bel[1, 1] = (torch.rand(1326, generator=g) < 0.01).float() * allowed[1]  # very sparse
    bel = bel / bel.sum(-1, keepdim=True).clamp(min=1e-30)
    potential = torch.randint(1, 2000, (rows, 2), generator=g)
    scale = torch.rand(rows, generator=g) * 1000 + 50
    tabs = showdown.BoardTables(boards.to(cuda_device))
    got = showdown.showdown_values(tabs, bel.to(cuda_device), potential, scale, table_of_row=table_of_row)
    want = oshow.showdown_values(boards.numpy()[table_of_row.numpy()], bel, potential, scale)
    torch.testing.assert_close(got.cpu(), want, rtol=RTOL, atol=ATOL)


def test_showdown_zero_sum_property(cuda_device):
    """Size-independent property: with potential = scale = 1 the belief-weighted values of
    the two players cancel (what one player wins the other loses)."""
    from poker2_b200 import showdown

    g = torch.Generator().manual_seed(9)
    m = 512
    boards = torch.stack([torch.randperm(52, generator=g)[:5] for _ in range(m)])
    allowed = torch.from_numpy(cards.allowed_mask(boards.numpy()))
    bel = torch.empty(m, 2, 1326).exponential_(generator=g) * allowed[:, None].float()
    bel = bel / bel.sum(-1, keepdim=True)
    tabs = showdown.BoardTables(boards.to(cuda_device))
    vals = showdown.showdown_values(tabs, bel.to(cuda_device), torch.ones(m, 2, dtype=torch.int64),
                                    torch.ones(m)).cpu().double()
    # weight each hand by its own probability and by the opponent mass it does not block
    from oracle import unblocked

    w0 = bel[:, 0].double() * unblocked.unblocked_mass(bel[:, 1]).double()
    w1 = bel[:, 1].double() * unblocked.unblocked_mass(bel[:, 0]).double()
    total = (vals[:, 0] * w0).sum(-1) + (vals[:, 1] * w1).sum(-1)
    assert total.abs().max().item() < 1e-5


def test_showdown_ev_from_sorted_inputs(cuda_device, golden_dir):
    """`showdown_ev_triton` (sorted-order inputs in, sorted-order EV out) against the sorted stage of the CPU
    oracle, which is pinned to upstream's `_showdown_value`: same bits on the golden boards, with the ranges of
    both players, a delta range, an all-zero range (den = 1, EV = 0 - 0) and a row of ties only."""
    from poker2_b200 import fused_cfr as F

    z = np.load(os.path.join(golden_dir, "showdown.npz"))
    boards = z["boards"][:8]
    bel = torch.from_numpy(z["beliefs"][:8])
    for x in (bel[:, 0], bel[:, 1]):
        x = x.clone()
        x[3] = 0.0
        first = int(np.flatnonzero(cards.allowed_mask(boards.astype(np.int64))[3])[17])
        x[3, first] = 1.0  # delta range
        x[5] = 0.0  # empty range
        st = oshow.sorted_ev(boards, x)
        got = F.showdown_ev_triton(st["b_sorted"].to(cuda_device).contiguous(), st["c1_sorted"].to(cuda_device),
                                   st["c2_sorted"].to(cuda_device), st["L"].to(cuda_device), st["R"].to(cuda_device))
        assert got.shape == st["ev_sorted"].shape and got.dtype == torch.float32
        diff = (got.cpu() - st["ev_sorted"]).abs().max().item()
        print("max abs difference", diff)
        assert torch.equal(got.cpu(), st["ev_sorted"])
    # one tie group over all positions: nobody wins or loses
    st = oshow.sorted_ev(boards[:1], bel[:1, 0])
    L, R = torch.zeros_like(st["L"]), torch.full_like(st["R"], 1326)
    got = F.showdown_ev_triton(st["b_sorted"].to(cuda_device).contiguous(), st["c1_sorted"].to(cuda_device),
                               st["c2_sorted"].to(cuda_device), L.to(cuda_device), R.to(cuda_device))
    assert got.abs().max().item() < 1e-6
    with pytest.raises(ValueError):
        F.showdown_ev_triton(st["b_sorted"], st["c1_sorted"], st["c2_sorted"], L, R)

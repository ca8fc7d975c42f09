"""The showdown and unblocked-mass oracles against values computed by the upstream code."""
import os

import numpy as np
import torch

from oracle import cards, showdown, unblocked


def test_showdown_oracle_bit_exact(golden_dir):
    z = np.load(os.path.join(golden_dir, "showdown.npz"))
    got = showdown.showdown_values(z["boards"], z["beliefs"], z["potential"], z["scale"])
    assert torch.equal(got, torch.from_numpy(z["values"]))


def test_sorted_stage_of_the_showdown_oracle_bit_exact(golden_dir):
    """`showdown.sorted_ev` (what the sorted-input kernel is checked against) composed with the inverse
    permutation, the hand mask and the pot scaling gives the upstream values."""
    z = np.load(os.path.join(golden_dir, "showdown.npz"))
    boards, bel = z["boards"][:6], torch.from_numpy(z["beliefs"][:6])
    allowed = torch.from_numpy(cards.allowed_mask(boards.astype(np.int64))).float()
    pot, scale = torch.from_numpy(z["potential"][:6]), torch.from_numpy(z["scale"][:6])
    for hero in range(2):
        st = showdown.sorted_ev(boards, bel[:, 1 - hero])
        ev = st["ev_sorted"].gather(1, torch.argsort(st["order"], dim=1)) * allowed
        got = ev * pot[:, hero][:, None] / scale[:, None]
        assert torch.equal(got, torch.from_numpy(z["values"][:6, hero]))


def test_showdown_oracle_against_enumeration(golden_dir):
    """Independent check: enumerate opponent hands for a handful of hero hands."""
    from oracle import rank7

    z = np.load(os.path.join(golden_dir, "showdown.npz"))
    b = 0
    board = z["boards"][b : b + 1]
    bel = torch.from_numpy(z["beliefs"][b : b + 1])
    vals = showdown.showdown_values(board, bel, np.ones((1, 2), dtype=np.int64), np.ones(1, dtype=np.float32))
    scores = rank7.rank_boards(board, rank7.MODE_PLANES)[0]
    ok = cards.allowed_mask(board.astype(np.int64))[0]
    compat = cards.compatible()
    opp = z["beliefs"][b, 1].astype(np.float64)
    for h in np.flatnonzero(ok)[::97]:
        w = opp * compat[h] * ok
        tot = w.sum()
        ev = ((w * (scores < scores[h])).sum() - (w * (scores > scores[h])).sum()) / tot
        assert abs(vals[0, 0, h].item() - ev) < 1e-5


def test_unblocked_oracle_bit_exact(golden_dir):
    z = np.load(os.path.join(golden_dir, "unblocked.npz"))
    got = unblocked.unblocked_mass(torch.from_numpy(z["x"]))
    assert torch.equal(got, torch.from_numpy(z["y"]))


def test_chance_oracle_matches_upstream_helper(golden_dir):
    """oracle/chance.py against ChanceNodeHelper.single_card_chance_values run upstream."""
    from oracle import chance as ochance

    z = np.load(os.path.join(golden_dir, "chance.npz"))
    w = torch.from_numpy(z["weights"])

    def value_fn(post, samples, lookup):
        newest = samples.gather(1, ((samples >= 0).sum(dim=1) - 1).view(-1, 1)).squeeze(1)
        scale = w[newest].view(-1, 1, 1)
        return torch.stack([post[:, 1], -post[:, 0]], dim=1) * scale + 0.25 * scale

    got = ochance.single_card_chance_values(torch.from_numpy(z["beliefs"]), torch.from_numpy(z["boards"]), value_fn)
    assert torch.equal(got, torch.from_numpy(z["expected"]))


def _flop_echo_model(z):
    cw, hw = torch.from_numpy(z["card_w"]), torch.from_numpy(z["hand_w"])

    def fn(post, boards, root):
        scale = cw.to(post.device)[boards[:, :3]].sum(dim=1).view(-1, 1, 1)
        return torch.stack([post[:, 1], -post[:, 0]], dim=1) * scale + hw.to(post.device).view(1, 1, -1) * 0.125

    return fn


def test_flop_chance_oracle_matches_upstream(golden_dir):
    """Canonical flops, suit-permutation table and both forms of flop_chance_values against the
    upstream helper (same generator seed for the sampled form)."""
    from oracle import flop_chance

    z = np.load(os.path.join(golden_dir, "flop_chance.npz"))
    canon, counts = flop_chance.canonical_flops()
    assert np.array_equal(canon, z["canonical"]) and np.array_equal(counts, z["counts"])
    assert np.array_equal(flop_chance.combo_perm(), z["combo_perm"].astype(np.int64))
    bel = torch.from_numpy(z["beliefs"])
    fn = _flop_echo_model(z)
    sampled = flop_chance.flop_chance_values(bel, fn, torch.Generator().manual_seed(int(z["sampled_seed"])))
    assert torch.equal(sampled, torch.from_numpy(z["sampled"]))
    exhaustive = flop_chance.flop_chance_values(bel, fn, None, sample_size=0, num_perm_samples=0)
    torch.testing.assert_close(exhaustive, torch.from_numpy(z["exhaustive"]), rtol=1e-6, atol=1e-7)

"""CUDA hand-ranking kernels (through the C ABI) against the oracle and the golden vectors."""
import os

import numpy as np
import pytest
import torch

from oracle import cards, rank7

pytestmark = pytest.mark.gpu


def _random_hands(n, seed):
    g = np.random.default_rng(seed)
    return np.argsort(g.random((n, 52)), axis=1)[:, :7].astype(np.int16)


def test_rank7_golden_bit_exact(cuda_device, golden_dir):
    from poker2_b200 import rules

    z = np.load(os.path.join(golden_dir, "rank7_hands.npz"))
    got = rules.rank_7_cards_single_batch(torch.from_numpy(z["hands"]).to(cuda_device))
    assert got.dtype == torch.int32
    assert np.array_equal(got.cpu().numpy(), z["packed"])


@pytest.mark.parametrize("n", [0, 1, 7, 1023, 1024, 1025, 200_003])
def test_rank7_random_vs_oracle(cuda_device, n):
    from poker2_b200 import rules

    hands = _random_hands(n, seed=n + 1)
    got = rules.rank_7_cards_single_batch(torch.from_numpy(hands).to(cuda_device)).cpu().numpy()
    assert np.array_equal(got, rank7.rank7(hands, rank7.MODE_IDS))
    if n:
        # any integer dtype is accepted, and an unaligned view takes the scalar-load path
        got64 = rules.rank_7_cards_single_batch(torch.from_numpy(hands.astype(np.int64)).to(cuda_device))
        assert np.array_equal(got64.cpu().numpy(), got)
        padded = torch.zeros(n * 7 + 1, dtype=torch.int16, device=cuda_device)
        padded[1:] = torch.from_numpy(hands).to(cuda_device).reshape(-1)
        view = padded[1:].view(n, 7)
        assert np.array_equal(rules.rank_7_cards_single_batch(view).cpu().numpy(), got)


def test_rank7_repeated_ids_follow_id_convention(cuda_device):
    from poker2_b200 import rules

    g = np.random.default_rng(5)
    hands = g.integers(0, 52, size=(50_000, 7)).astype(np.int16)  # repeats are common
    got = rules.rank_7_cards_single_batch(torch.from_numpy(hands).to(cuda_device)).cpu().numpy()
    assert np.array_equal(got, rank7.rank7(hands, rank7.MODE_IDS))


def test_all_flush_and_straight_masks(cuda_device):
    """Every 5..7-card subset of one suit, and every rank set with 5..7 distinct ranks."""
    from itertools import combinations

    from poker2_b200 import rules

    hands = []
    for k in (5, 6, 7):
        for ranks in combinations(range(13), k):
            suited = [r for r in ranks]  # suit 0
            filler = [13 + r for r in range(13) if r not in ranks][: 7 - k]
            hands.append(suited + [f + 13 * (i % 2) for i, f in enumerate(filler)])
            rainbow = [r + 13 * (i % 4) for i, r in enumerate(ranks)]
            pad = [r + 13 * ((i + 1) % 4) for i, r in enumerate(ranks)][: 7 - k]
            hands.append(rainbow + pad)
    hands = np.asarray(hands, dtype=np.int16)
    got = rules.rank_7_cards_single_batch(torch.from_numpy(hands).to(cuda_device)).cpu().numpy()
    assert np.array_equal(got, rank7.rank7(hands, rank7.MODE_IDS))


def test_compare_entry_points(cuda_device, golden_dir):
    from poker2_b200 import rules

    z = np.load(os.path.join(golden_dir, "rules_known_answers.npz"))
    a = torch.from_numpy(z["a"]).to(cuda_device)
    b = torch.from_numpy(z["b"]).to(cuda_device)
    got = rules.compare_7_batches(a, b)
    assert np.array_equal(got.cpu().numpy(), z["result"])

    # the upstream GPU test: 2048 seeded random pairs, planes and card ids agree
    g = torch.Generator().manual_seed(1234)
    cards_batch = torch.stack([torch.stack([torch.randperm(52, generator=g)[:7] for _ in range(2)])
                               for _ in range(2048)])
    planes = torch.zeros(2048, 2, 4, 13, dtype=torch.bool)
    for p in range(2):
        for j in range(7):
            c = cards_batch[:, p, j]
            planes[torch.arange(2048), p, c // 13, c % 13] = True
    want = rank7.compare7(cards_batch.numpy(), rank7.MODE_PLANES)
    assert np.array_equal(rules.compare_7_single_batch(planes.to(cuda_device)).cpu().numpy(), want)
    assert np.array_equal(rules.compare_7_cards_single_batch(cards_batch.to(cuda_device)).cpu().numpy(), want)


def test_rank_hands_order_and_groups(cuda_device, golden_dir):
    from poker2_b200 import rules

    z = np.load(os.path.join(golden_dir, "rank_hands.npz"))
    boards = torch.from_numpy(z["boards"]).to(cuda_device)
    scores, order = rules.rank_hands(boards)
    assert scores.dtype == torch.int32 and order.dtype == torch.int64
    scores, order = scores.cpu().numpy(), order.cpu().numpy()
    want_scores, want_order = rank7.rank_hands(z["boards"], rank7.MODE_IDS)
    assert np.array_equal(scores, want_scores)
    assert np.array_equal(order, want_order)
    # on combos that do not touch the board, order and tie groups equal the upstream ones
    ok = cards.allowed_mask(z["boards"].astype(np.int64))
    for b in range(len(z["boards"])):
        mine = [h for h in order[b] if ok[b, h]]
        theirs = [h for h in z["order"][b].astype(np.int64) if ok[b, h]]
        assert mine == theirs
        dense = z["dense"][b]
        s = scores[b]
        idx = np.flatnonzero(ok[b])
        same_mine = s[idx][:, None] == s[idx][None, :]
        same_theirs = dense[idx][:, None] == dense[idx][None, :]
        assert np.array_equal(same_mine, same_theirs)


def test_argument_errors(cuda_device):
    from poker2_b200 import rules

    with pytest.raises(ValueError):
        rules.rank_7_cards_single_batch(torch.zeros(4, 6, dtype=torch.int16, device=cuda_device))
    with pytest.raises(ValueError):
        rules.rank_7_cards_single_batch(torch.zeros(4, 7, dtype=torch.int16))
    with pytest.raises(ValueError):
        rules.compare_7_single_batch(torch.zeros(4, 2, 4, 12, dtype=torch.bool, device=cuda_device))
    with pytest.raises(ValueError):
        rules.rank_hands(torch.zeros(4, 4, dtype=torch.int64, device=cuda_device))
    with pytest.raises(ValueError):
        rules.compare_7_batches(torch.zeros(2, 4, 13), torch.zeros(3, 4, 13))


def test_rank7_every_count_pattern(cuda_device):
    """Hands drawn per rank-multiplicity pattern (4+3, 4+2+1, 3+3+1, 3+2+2, 2+2+2+1, ...),
    so that the rare hand types are as frequent as the common ones."""
    from poker2_b200 import rules

    g = np.random.default_rng(11)
    patterns = [(4, 3), (4, 2, 1), (4, 1, 1, 1), (3, 3, 1), (3, 2, 2), (3, 2, 1, 1), (3, 1, 1, 1, 1), (2, 2, 2, 1),
                (2, 2, 1, 1, 1), (2, 1, 1, 1, 1, 1), (1, 1, 1, 1, 1, 1, 1)]
    hands = []
    for pat in patterns:
        for _ in range(4000):
            ranks = g.choice(13, size=len(pat), replace=False)
            hand = []
            for r, cnt in zip(ranks, pat):
                hand += [int(s) * 13 + int(r) for s in g.choice(4, size=cnt, replace=False)]
            g.shuffle(hand)
            hands.append(hand)
    hands = np.asarray(hands, dtype=np.int16)
    got = rules.rank_7_cards_single_batch(torch.from_numpy(hands).to(cuda_device)).cpu().numpy()
    assert np.array_equal(got, rank7.rank7(hands, rank7.MODE_IDS))

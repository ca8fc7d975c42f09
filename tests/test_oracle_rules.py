"""The C hand-rank oracle against golden vectors produced by the upstream evaluator."""
import os

import numpy as np

from oracle import rank7


def _planes_to_cards(planes):
    # [K,4,13] 0/1 -> list of card-id arrays (7 cards each in the recorded cases)
    out = []
    for p in planes:
        s, r = np.nonzero(p)
        out.append((s * 13 + r).astype(np.int16))
    return out


def test_recorded_upstream_comparisons(golden_dir):
    z = np.load(os.path.join(golden_dir, "rules_known_answers.npz"))
    assert len(z["result"]) >= 40
    assert np.array_equal(rank7.compare_planes(z["a"], z["b"]), z["result"])
    # the card-id entry point agrees wherever both hands really hold seven cards
    a, b = _planes_to_cards(z["a"]), _planes_to_cards(z["b"])
    for mode in (rank7.MODE_PLANES, rank7.MODE_IDS):
        for ca, cb, want in zip(a, b, z["result"]):
            if len(ca) == 7 and len(cb) == 7:
                assert rank7.compare7(np.stack([ca, cb])[None], mode)[0] == want


def test_packed_scores_match_upstream(golden_dir):
    z = np.load(os.path.join(golden_dir, "rank7_hands.npz"))
    for mode in (rank7.MODE_PLANES, rank7.MODE_IDS):
        assert np.array_equal(rank7.rank7(z["hands"], mode), z["packed"])


def test_corner_case_fields(golden_dir):
    z = np.load(os.path.join(golden_dir, "rank7_hands.npz"))
    packed = z["packed"][: int(z["num_corner"])]
    fields = [[(p >> s) & 15 for s in (20, 16, 12, 8, 4, 0)] for p in packed]
    assert fields[0] == [5, 1, 0, 0, 0, 0]  # lowest window of a six-card straight
    assert fields[1] == [5, 0, 0, 0, 0, 0]  # wheel preferred over the 6-high straight
    assert fields[2] == [8, 6, 1, 0, 0, 0]  # quads kicker = the pair, not the ace
    assert fields[3] == [3, 12, 11, 0, 0, 0]  # third pair outranks the queen kicker
    assert fields[4] == [9, 5, 0, 0, 0, 0]  # highest window of a six-card straight flush
    assert fields[5] == [7, 7, 5, 0, 0, 0]


def test_board_ranking_matches_upstream_order_and_groups(golden_dir):
    z = np.load(os.path.join(golden_dir, "rank_hands.npz"))
    scores, order = rank7.rank_hands(z["boards"], rank7.MODE_PLANES)
    assert np.array_equal(order, z["order"].astype(np.int64))
    for b in range(scores.shape[0]):
        s = scores[b][order[b]]
        gid = np.cumsum(np.concatenate([[1], (s[1:] != s[:-1]).astype(np.int64)]))
        dense = np.empty(1326, dtype=np.int64)
        dense[order[b]] = gid
        assert np.array_equal(dense, z["dense"][b])


def test_id_mode_agrees_on_unblocked_combos(golden_dir):
    from oracle import cards

    z = np.load(os.path.join(golden_dir, "rank_hands.npz"))
    planes = rank7.rank_boards(z["boards"], rank7.MODE_PLANES)
    ids = rank7.rank_boards(z["boards"], rank7.MODE_IDS)
    ok = cards.allowed_mask(z["boards"].astype(np.int64))
    assert np.array_equal(planes[ok], ids[ok])
    assert ok.sum(axis=1).tolist() == [1081] * len(z["boards"])

"""Generates the golden vectors under tests/golden/ by RUNNING THE UPSTREAM P2 CODE.

Run it on a machine where the upstream checkout is mounted, with P2_REFERENCE_SRC set to
its `src` directory and P2_REFERENCE_TESTS to its `tests` directory:

    P2_REFERENCE_SRC=<checkout>/src P2_REFERENCE_TESTS=<checkout>/tests \
        python tests/golden/make_golden.py [section ...]

Sections (default: all): rules, showdown, unblocked, tree, cfr, turn, training_data, warm_start, chance, flop_chance,
replay, rounds, steps, production, standard, zero_sum, ragged256, cfr_avg, running_values, warm_br, linear,
policy_head, dataclass_defaults, policy_delta, depth5,
default_bins.  The outputs are small .npz files that travel with the repository;
the test-suite reads only those files, never the upstream checkout.
"""
from __future__ import annotations

import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import refshim  # noqa: E402

refshim.install()

import numpy as np  # noqa: E402
import torch  # noqa: E402

REF_TESTS = os.environ.get("P2_REFERENCE_TESTS") or os.path.join(
    os.path.dirname(os.environ.get("P2_REFERENCE_SRC", "").rstrip("/")), "tests")


def save(name: str, **arrays) -> None:
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **arrays)
    print(f"wrote {path} ({os.path.getsize(path) / 1024:.1f} KiB)")


def pack_fields(cv: torch.Tensor) -> torch.Tensor:
    off = 4 * (5 - torch.arange(6, dtype=torch.int))
    return (cv.to(torch.int) << off).sum(dim=-1)


def cards_to_planes(hands: torch.Tensor) -> torch.Tensor:
    n = hands.shape[0]
    planes = torch.zeros(n, 1, 4, 13, dtype=torch.int)
    for j in range(hands.shape[1]):
        planes[torch.arange(n), 0, hands[:, j] // 13, hands[:, j] % 13] = 1
    return planes


# --------------------------------------------------------------------------------------
def gen_rules() -> None:
    import pytest
    from p2.env import rules

    # (1) every comparison the upstream test-suite makes, recorded while its tests run
    recorded = []
    original = rules.compare_7_batches

    def recorder(a, b):
        res = original(a, b)
        recorded.append((a.clone(), b.clone(), res.clone()))
        return res

    rules.compare_7_batches = recorder
    try:
        rc = pytest.main(["-q", "-p", "no:cacheprovider", "-x", os.path.join(REF_TESTS, "test_rules.py")])
    finally:
        rules.compare_7_batches = original
    assert rc == 0, "upstream tests/test_rules.py must pass before its cases are recorded"
    a = torch.cat([r[0] for r in recorded]).to(torch.int8).numpy()
    b = torch.cat([r[1] for r in recorded]).to(torch.int8).numpy()
    res = torch.cat([r[2] for r in recorded]).to(torch.int32).numpy()
    save("rules_known_answers.npz", a=a, b=b, result=res)

    # (2) packed scores of hand-built corner cases and of seeded random hands
    def C(r, s):
        return s * 13 + r

    corner = [
        [C(0, 0), C(1, 1), C(2, 2), C(3, 3), C(4, 0), C(5, 1), C(11, 2)],  # six-card straight
        [C(12, 0), C(0, 1), C(1, 2), C(2, 3), C(3, 0), C(4, 1), C(9, 2)],  # wheel and 6-high
        [C(6, 0), C(6, 1), C(6, 2), C(6, 3), C(1, 0), C(1, 1), C(12, 2)],  # quads + pair + ace
        [C(12, 0), C(12, 1), C(11, 0), C(11, 1), C(0, 2), C(0, 3), C(10, 2)],  # three pairs
        [C(3, 3), C(4, 3), C(5, 3), C(6, 3), C(7, 3), C(8, 3), C(0, 0)],  # six-card straight flush
        [C(7, 0), C(7, 1), C(7, 2), C(5, 0), C(5, 1), C(5, 2), C(12, 3)],  # two trips
        [C(12, 0), C(10, 1), C(8, 2), C(6, 3), C(4, 0), C(2, 1), C(0, 2)],  # no pair
        [C(12, 1), C(11, 1), C(7, 1), C(5, 1), C(3, 1), C(1, 1), C(4, 0)],  # six-card flush
        [C(12, 2), C(0, 2), C(1, 2), C(2, 2), C(3, 2), C(8, 0), C(8, 1)],  # steel wheel + pair
        [C(12, 0), C(11, 0), C(10, 0), C(9, 0), C(8, 0), C(8, 1), C(8, 2)],  # royal + trips
        [C(4, 0), C(4, 1), C(4, 2), C(9, 0), C(9, 1), C(2, 3), C(3, 3)],  # full house
        [C(0, 0), C(0, 1), C(0, 2), C(0, 3), C(12, 0), C(12, 1), C(12, 2)],  # quads + trips
        [C(8, 0), C(9, 1), C(10, 2), C(11, 3), C(12, 0), C(0, 1), C(1, 2)],  # broadway
        [C(2, 0), C(2, 1), C(5, 2), C(5, 3), C(9, 0), C(10, 1), C(12, 2)],  # two pair, ace kicker
    ]
    g = torch.Generator().manual_seed(1234)
    rand = torch.stack([torch.randperm(52, generator=g)[:7] for _ in range(8192)])
    hands = torch.cat([torch.tensor(corner), rand])
    packed = pack_fields(rules.create_comparison_vector(cards_to_planes(hands))[:, 0])
    save("rank7_hands.npz", hands=hands.to(torch.int16).numpy(), packed=packed.numpy().astype(np.int32),
         num_corner=np.int64(len(corner)))

    # (3) per-board ranking of all 1326 combos (dense group ids and stable order)
    boards = torch.stack([torch.randperm(52, generator=g)[:5] for _ in range(12)])
    boards[0] = torch.tensor([C(12, 0), C(11, 0), C(10, 0), C(9, 0), C(8, 0)])  # royal flush on board
    boards[1] = torch.tensor([C(1, 0), C(2, 0), C(3, 0), C(7, 1), C(12, 1)])
    boards[2] = torch.tensor([C(5, 0), C(5, 1), C(5, 2), C(9, 3), C(9, 0)])  # full house on board
    dense, order = rules.rank_hands(boards)
    save("rank_hands.npz", boards=boards.to(torch.int16).numpy(), dense=dense.numpy().astype(np.int32),
         order=order.numpy().astype(np.int16))


# --------------------------------------------------------------------------------------
def dirichlet_ranges(boards: torch.Tensor, g: torch.Generator, alpha: float = 1.0) -> torch.Tensor:
    """[M,2,1326] ranges ~ Dirichlet(alpha) over the combos not blocked by the board."""
    from p2.env.card_utils import combo_to_onehot_tensor

    onehot = combo_to_onehot_tensor().float()
    m = boards.shape[0]
    board_mask = torch.zeros(m, 52)
    board_mask.scatter_(1, boards.clamp(min=0), (boards >= 0).float())
    allowed = (onehot @ board_mask.T).T < 0.5
    if alpha == 1.0:
        gam = torch.empty(m, 2, 1326).exponential_(generator=g)
    else:
        gam = torch.distributions.Gamma(alpha, 1.0).sample((m, 2, 1326))
    gam = gam * allowed[:, None, :]
    return gam / gam.sum(-1, keepdim=True)


def gen_showdown() -> None:
    from p2.search.sparse_cfr_evaluator import SparseCFREvaluator

    g = torch.Generator().manual_seed(7)
    m = 8
    boards = torch.stack([torch.randperm(52, generator=g)[:5] for _ in range(m)])
    boards[1] = torch.tensor([12, 11, 10, 9, 8])
    boards[2] = torch.tensor([0, 13, 26, 5, 18])
    boards[3] = torch.tensor([3, 16, 7, 20, 12 + 26])
    beliefs = dirichlet_ranges(boards, g)
    # a range concentrated on three hands, and a uniform one
    allowed3 = torch.where(beliefs[4, 0] > 0)[0]
    beliefs[4, 0] = 0
    beliefs[4, 0, allowed3[:3]] = torch.tensor([0.5, 0.25, 0.25])
    beliefs[5, 1] = (beliefs[5, 1] > 0).float() / (beliefs[5, 1] > 0).sum()
    potential = torch.randint(10, 600, (m, 2), generator=g)
    scale = (torch.rand(m, generator=g) * 900 + 100).float()

    from p2.env.card_utils import combo_to_onehot_tensor

    onehot = combo_to_onehot_tensor().float()
    board_mask = torch.zeros(m, 52)
    board_mask.scatter_(1, boards, 1.0)
    ev = SparseCFREvaluator.__new__(SparseCFREvaluator)
    ev.device = torch.device("cpu")
    ev.showdown_indices = torch.arange(m)
    ev.env = types.SimpleNamespace(board_indices=boards, scale=scale)
    ev.allowed_hands = (onehot @ board_mask.T).T < 0.5
    ev.showdown_potential = potential
    ev._init_hand_rank_data()
    values = ev._showdown_value_both(beliefs)
    save("showdown.npz", boards=boards.to(torch.int16).numpy(), beliefs=beliefs.numpy(),
         potential=potential.numpy(), scale=scale.numpy(), values=values.numpy())


def gen_unblocked() -> None:
    from p2.env.card_utils import calculate_unblocked_mass

    g = torch.Generator().manual_seed(11)
    x = torch.rand(6, 1326, generator=g)
    x[1] = 0
    x[1, 100] = 1.0  # delta
    x[2] = 1.0 / 1326  # uniform
    x[3] = x[3] * (torch.rand(1326, generator=g) < 0.05)  # sparse
    save("unblocked.npz", x=x.numpy(), y=calculate_unblocked_mass(x).numpy())


SECTIONS = {"rules": gen_rules, "showdown": gen_showdown, "unblocked": gen_unblocked}

if __name__ == "__main__":
    try:
        import golden_cfr  # noqa: F401  (registers the tree and cfr sections)

        import golden_replay  # noqa: F401  (registers replay)
        import golden_rounds  # noqa: F401  (registers rounds)
        import golden_steps  # noqa: F401  (registers steps)
        import golden_settings  # noqa: F401  (registers production, standard, zero_sum, ragged256)

        SECTIONS.update(golden_cfr.SECTIONS)
    except ImportError:
        pass
    wanted = sys.argv[1:] or list(SECTIONS)
    for name in wanted:
        print(f"== {name}")
        SECTIONS[name]()

"""Host tree builder and the CFR oracle against arrays produced by the upstream evaluator."""
import os

import numpy as np
import pytest
import torch

from leaf_models import pot_echo_leaf_fn
from oracle import cfr as ocfr
from poker2_b200 import tree as ptree

BET_BINS = [0.5, 1.0]


def _build(pot, stack, cap, depth):
    roots = ptree.root_states(pot, stack, min_raise=2)
    return ptree.build_trees(roots, BET_BINS, depth, bb=2, max_raises=cap)


@pytest.mark.parametrize("tag,cap", [("cap2", 2), ("nocap", None)])
def test_tree_indices_and_legal_masks_bit_exact(golden_dir, tag, cap):
    z = np.load(os.path.join(golden_dir, "tree.npz"))
    t = _build(z["pots"], z["stacks"], cap, int(z[f"{tag}_max_depth"]))
    assert t.depth_offsets == z[f"{tag}_depth_offsets"].tolist()
    for name, mine in [
        ("parent_index", t.parent_index), ("action_from_parent", t.action_from_parent), ("to_act", t.state.to_act),
        ("legal_mask", t.legal_mask), ("leaf_mask", t.leaf_mask), ("child_count", t.child_count),
        ("child_offsets", t.child_offsets), ("done", t.state.done), ("street", t.state.street),
        ("pot", t.state.pot), ("stacks", t.state.stacks), ("showdown_potential", t.showdown_potential),
        ("scale", t.state.scale), ("prev_actor", t.prev_actor), ("fold_value", t.fold_value),
    ]:
        assert np.array_equal(mine, z[f"{tag}_{name}"]), name


def _oracle_from_golden(z):
    cap = int(z["cap"])
    t = _build(z["pot"], z["stack"], None if cap < 0 else cap, int(z["max_depth"]))
    assert t.total_nodes == int(z["total_nodes"])
    o = ocfr.SubgameOracle(t.oracle_dict(z["boards"].astype(np.int64)), torch.from_numpy(z["ranges"]),
                           iterations=int(z["iterations"]))
    return o.solve()


def test_cfr_oracle_bit_exact_short_run(golden_dir):
    z = np.load(os.path.join(golden_dir, "cfr_single_cap2_t8.npz"))
    o = _oracle_from_golden(z)
    assert torch.equal(o.policy, torch.from_numpy(z["policy"]))
    assert torch.equal(o.regrets, torch.from_numpy(z["regrets"]))
    assert torch.equal(o.weight_sums, torch.from_numpy(z["weight_sums"]))
    assert torch.equal(o.beliefs, torch.from_numpy(z["beliefs"]))
    assert torch.equal(o.policy_avg, torch.from_numpy(z["policy_avg"]))
    assert torch.equal(o.values_avg, torch.from_numpy(z["values_avg"]))
    ex, br = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["exploitability"]))
    assert torch.equal(br, torch.from_numpy(z["br_values"]))


@pytest.mark.parametrize("name", ["cfr_single_nocap_t32", "cfr_batch_cap2_t24"])
def test_cfr_oracle_bit_exact_other_trees(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    o = _oracle_from_golden(z)
    assert torch.equal(o.policy_avg, torch.from_numpy(z["policy_avg"]))
    assert torch.equal(o.values_avg[: o.N], torch.from_numpy(z["root_values"]))
    ex, _ = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["exploitability"]))


def _turn_trees(z):
    roots = ptree.root_states(z["pot"], z["stack"], min_raise=2, street=2)
    return ptree.build_trees(roots, BET_BINS, int(z["max_depth"]), bb=2, max_raises=int(z["cap"]))


def test_turn_tree_matches_upstream(golden_dir):
    z = np.load(os.path.join(golden_dir, "cfr_turn_cap2_t16.npz"))
    t = _turn_trees(z)
    assert t.total_nodes == int(z["total_nodes"])
    assert np.array_equal(t.parent_index, z["parent_index"])
    assert np.array_equal(t.leaf_mask, z["leaf_mask"])
    assert np.array_equal(t.state.street, z["street"])
    assert np.array_equal(t.leaf_mask & ~t.state.done, z["model_mask"])


def test_cfr_oracle_with_model_leaves_bit_exact(golden_dir):
    """Turn subgames whose non-fold leaves are valued by a stand-in model, against the
    upstream evaluator run with the same model."""
    z = np.load(os.path.join(golden_dir, "cfr_turn_cap2_t16.npz"))
    t = _turn_trees(z)
    boards = np.concatenate([z["boards"].astype(np.int64), np.full((z["boards"].shape[0], 1), -1)], axis=1)
    w = torch.from_numpy(z["hand_weights"])

    def leaf_fn(beliefs, idx):
        return pot_echo_leaf_fn(t, idx, w)(beliefs)

    o = ocfr.SubgameOracle(t.oracle_dict(boards), torch.from_numpy(z["ranges"]), iterations=int(z["iterations"]),
                           leaf_fn=leaf_fn).solve()
    assert torch.equal(o.regrets, torch.from_numpy(z["regrets"]))
    assert torch.equal(o.policy_avg, torch.from_numpy(z["policy_avg"]))
    assert torch.equal(o.values_avg[: o.N], torch.from_numpy(z["root_values"]))
    ex, br = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["exploitability"]))
    assert torch.equal(br, torch.from_numpy(z["br_values"]))


def test_sampling_schedule_matches_upstream(golden_dir):
    from poker2_b200 import sampling

    z = np.load(os.path.join(golden_dir, "cfr_turn_cap2_t16.npz"))
    got = sampling.sampling_schedule(3, int(z["iterations"]), torch.Generator().manual_seed(99))
    assert np.array_equal(got.numpy(), z["schedule_seed99"])


def test_sample_leaves_matches_upstream(golden_dir):
    """The walk from the roots to the next public states, with the upstream run's sampling
    policy and beliefs and the same generator seed, lands on the same states."""
    from poker2_b200 import sampling

    z = np.load(os.path.join(golden_dir, "cfr_turn_cap2_t16.npz"))
    t = _turn_trees(z)
    nodes, cont, bel = sampling.sample_leaves(
        t, torch.from_numpy(z["policy_sample"]), torch.from_numpy(z["beliefs_last"]),
        torch.Generator().manual_seed(321), sample_epsilon=float(z["sample_epsilon"]), training_mode=True)
    assert torch.equal(bel, torch.from_numpy(z["sampled_beliefs"]))
    assert np.array_equal(t.state.pot[cont.numpy()], z["sampled_pot"])
    assert np.array_equal(t.state.stacks[cont.numpy()], z["sampled_stacks"])


def test_layout_rejects_trees_beyond_the_kernel_limits():
    """Host-side guard: subgames with more nodes than the kernels hold are refused before any launch."""
    from poker2_b200 import solver

    roots = ptree.root_states(np.array([100]), np.array([8000]), min_raise=2)
    big = ptree.build_trees(roots, [0.25, 0.5, 1.0], 10, bb=2)  # three bet sizes, no raise cap
    assert big.total_nodes > solver.MAX_NODES
    with pytest.raises(ValueError, match="nodes"):
        solver.device_layout(big, np.array([[0, 1, 2, 3, 4]]))
    small = ptree.build_trees(roots, [0.5, 1.0], 8, bb=2, max_raises=2)
    layout = solver.device_layout(small, np.array([[0, 1, 2, 3, 4]]))
    assert layout.rows == small.total_nodes and layout.num_model_leaves == 0
    # one root, ragged batch of one: offsets and records are consistent
    assert layout.subgames[0]["n_nodes"] == small.total_nodes
    assert int(solver.node_kind(layout.nodes)[0]) == ptree.KIND_INTERNAL and int(solver.node_to_act(layout.nodes)[0]) in (0, 1)


def test_cfr_oracle_warm_start_bit_exact(golden_dir):
    """Start policy from a policy head and regrets seeded from it (warm start of type `model`),
    against the upstream evaluator."""
    z = np.load(os.path.join(golden_dir, "cfr_warm_cap2_t12.npz"))
    t = _build(z["pot"], z["stack"], int(z["cap"]), int(z["max_depth"]))
    assert t.total_nodes == int(z["total_nodes"])
    o = ocfr.SubgameOracle(t.oracle_dict(z["boards"].astype(np.int64)), torch.from_numpy(z["ranges"]),
                           iterations=int(z["iterations"]), start_policy=torch.from_numpy(z["start_policy"]),
                           warm_start_iterations=int(z["warm_start_iterations"]),
                           warm_start_multiplier=float(z["warm_start_multiplier"]))
    o.initialize()
    o.warm_start()
    assert torch.equal(o.regrets, torch.from_numpy(z["seeded_regrets"]))
    assert torch.equal(o.weight_sums, torch.from_numpy(z["seeded_weights"]))
    for tt in range(o.warm_start_iterations, o.iterations):
        o.iteration(tt)
    o.finalize()
    assert torch.equal(o.regrets, torch.from_numpy(z["regrets"]))
    assert torch.equal(o.policy_avg, torch.from_numpy(z["policy_avg"]))
    assert torch.equal(o.values_avg[: o.N], torch.from_numpy(z["root_values"]))
    ex, _ = o.exploitability()
    assert torch.equal(ex, torch.from_numpy(z["exploitability"]))


@pytest.mark.parametrize("cfr_type", ["standard", "linear", "discounted", "discounted_plus"])
def test_iteration_scalars_follow_the_oracle_schedule(cfr_type):
    """The per-pass records the kernels read against the oracle's own schedule functions: mixing
    weights (`_get_mixing_weights`, cfr_evaluator.py:285-303), the pass that only copies the policy
    (:1197-1205) and, for linear CFR, the player whose actions take no regret (:1348-1349)."""
    from poker2_b200 import solver

    iterations, delay = 9, 3
    sc = solver.iteration_scalars(iterations, cfr_type=cfr_type, alpha=1.5, beta=0.5, gamma=2.0, dcfr_delay=delay)
    o = ocfr.SubgameOracle.__new__(ocfr.SubgameOracle)
    o.cfr_type, o.gamma, o.dcfr_delay = cfr_type, 2.0, delay
    for t in range(iterations):
        old, new = o.mixing_weights(t)
        assert sc[t]["mix_old"] == np.float32(old) and sc[t]["mix_new"] == np.float32(new)
        assert sc[t]["mix_total"] == np.float32(old + new)
        copies = t == 0 or (cfr_type in ("discounted", "discounted_plus") and t <= delay)
        assert (int(sc[t]["do_mix"]) & 1) == (0 if copies else 1)
        skipped = (int(sc[t]["do_mix"]) >> 1) & 3
        assert skipped == ((t % 2) + 1 if cfr_type == "linear" else 0)
        if cfr_type in ("discounted", "discounted_plus"):
            assert sc[t]["num_pos"] == np.float32(t ** 1.5) and sc[t]["den_pos"] == np.float32(t ** 1.5 + 1)
            assert sc[t]["num_neg"] == np.float32(t ** 0.5) and sc[t]["den_neg"] == np.float32(t ** 0.5 + 1)
        else:
            assert sc[t]["num_pos"] == sc[t]["den_pos"] == sc[t]["num_neg"] == sc[t]["den_neg"] == 1.0
    assert solver.scalars_are_linear(sc) == (cfr_type == "linear")

"""The evaluator facade (initialize_subgame / evaluate_cfr / training_data) against the
batches the upstream evaluator returned for the same river subgames."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_training_data_matches_upstream(cuda_device, golden_dir):
    from poker2_b200 import evaluator, tree as ptree

    z = np.load(os.path.join(golden_dir, "training_data_cap2_t12.npz"))
    roots = ptree.root_states(z["pot"], z["stack"], min_raise=2)
    env = evaluator.env_view(roots, z["boards"].astype(np.int64))
    w = torch.from_numpy(z["hand_weights"]).to(cuda_device)

    def model(beliefs, boards, context):
        # the stand-in network of the golden run (tests/golden/golden_cfr.py, PotEchoModel)
        sw = (0.5 + context[:, 0].clamp(0.0, 10.0)).view(-1, 1) * w.view(1, 1326)
        return torch.stack([sw + beliefs[:, 1], sw * (-0.5) + beliefs[:, 0]], dim=1)

    ev = evaluator.SubgameEvaluator(cuda_device, iterations=int(z["iterations"]), max_depth=int(z["max_depth"]),
                                    max_raises=int(z["cap"]), generator=torch.Generator().manual_seed(0), model=model)
    ev.initialize_subgame(env, torch.arange(2), torch.from_numpy(z["ranges"]))
    assert ev.root_nodes == 2 and ev.stats["evaluator_root_nodes"] == 2.0
    sampled = ev.evaluate_cfr(training_mode=True)
    assert sampled.beliefs.shape[1:] == (2, 1326) and len(sampled.nodes) == sampled.beliefs.shape[0]
    value_batch, pre_batch, policy_batch = ev.training_data(exclude_start=True)
    # roots at the start of the river round: targets averaged over the 48 possible river cards
    assert len(pre_batch) == int(z["pre_count"])
    close = lambda a, b: torch.testing.assert_close(a.cpu(), torch.from_numpy(b), rtol=1e-5, atol=1e-6)  # noqa: E731
    close(value_batch.value_targets, z["value_targets"])
    close(value_batch.beliefs, z["value_beliefs"])
    close(policy_batch.policy_targets, z["policy_targets"])
    close(policy_batch.beliefs, z["policy_beliefs"])
    close(pre_batch.value_targets, z["pre_value_targets"])
    close(pre_batch.beliefs, z["pre_beliefs"])
    for key in ("board", "street", "stage"):
        assert np.array_equal(pre_batch.statistics[key].cpu().numpy(), z["pre_" + key]), key
    close(value_batch.statistics["local_exploitability"], z["value_exploitability"])
    close(value_batch.statistics["local_best_response_values"], z["value_br"])
    for got, want in [(value_batch.legal_masks, "value_legal_masks"), (policy_batch.legal_masks, "policy_legal_masks"),
                      (value_batch.statistics["pot"], "value_pot"), (policy_batch.statistics["pot"], "policy_pot"),
                      (value_batch.statistics["to_act"], "value_to_act"),
                      (policy_batch.statistics["to_act"], "policy_to_act"),
                      (value_batch.statistics["bet_amounts"], "value_bet_amounts"),
                      (policy_batch.statistics["bet_amounts"], "policy_bet_amounts")]:
        assert np.array_equal(got.cpu().numpy(), z[want]), want


def test_evaluator_with_warm_start(cuda_device, golden_dir):
    """With warm-start iterations of type `model` the facade still solves terminal-leaf trees through the
    one-call solve (uniform start policy when none is given) and returns well-formed batches."""
    from poker2_b200 import evaluator, solver, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_warm_cap2_t12.npz"))
    roots = ptree.root_states(z["pot"], z["stack"], min_raise=2)
    env = evaluator.env_view(roots, z["boards"].astype(np.int64))
    ev = evaluator.SubgameEvaluator(cuda_device, iterations=int(z["iterations"]), max_depth=int(z["max_depth"]),
                                    max_raises=int(z["cap"]), generator=torch.Generator().manual_seed(5),
                                    warm_start_iterations=int(z["warm_start_iterations"]),
                                    warm_start_multiplier=float(z["warm_start_multiplier"]))
    ev.initialize_subgame(env, torch.arange(2), torch.from_numpy(z["ranges"]))
    assert not isinstance(ev.solver, solver.SteppedSolver)
    ev.evaluate_cfr(start_policy=torch.from_numpy(z["start_policy"]))
    value_batch, _, policy_batch = ev.training_data()
    torch.testing.assert_close(value_batch.value_targets.cpu(), torch.from_numpy(z["root_values"]).clamp(-1, 1),
                               rtol=1e-5, atol=1e-6)
    assert np.array_equal(ev.t_sample.numpy(), z["t_sample"])  # same generator seed as the upstream run
    # the solver state under the upstream attribute names, upstream node order
    n = ev.root_nodes
    close = lambda a, b: torch.testing.assert_close(a.cpu(), torch.from_numpy(b), rtol=1e-5, atol=1e-6)  # noqa: E731
    close(ev.cumulative_regrets[n:], z["regrets"][n:])
    close(ev.regret_weight_sums[n:], z["weight_sums"][n:])
    close(ev.policy_probs_avg[n:], z["policy_avg"][n:])
    close(ev.policy_probs_sample[n:], z["policy_sample"][n:])
    assert ev.values_avg.shape == (int(z["total_nodes"]), 2, 1326) and ev.beliefs.shape == ev.values_avg.shape
    assert ev.depth_offsets[-1] == int(z["total_nodes"]) and ev.parent_index.shape[0] == int(z["total_nodes"])
    assert int(ev.child_count.sum()) == int(z["total_nodes"]) - n and ev.legal_mask.shape[1] == 5
    ev.evaluate_cfr()  # uniform start policy
    value_batch, _, policy_batch = ev.training_data()
    assert torch.isfinite(value_batch.value_targets).all() and torch.isfinite(policy_batch.policy_targets).all()


def test_evaluator_on_flop_subgames_with_network_leaves(cuda_device):
    """Flop roots: leaves at the start of the turn valued by a small network averaged over the
    49 turn cards, and a pre-chance batch averaged over the canonical flops."""
    from poker2_b200 import evaluator, leaf_eval, tree as ptree

    g = torch.Generator().manual_seed(8)
    n = 2
    boards = torch.full((n, 5), -1, dtype=torch.int64)
    for i in range(n):
        boards[i, :3] = torch.randperm(52, generator=g)[:3]
    pot, stack = np.array([40, 90]), np.array([400, 250])
    roots = ptree.root_states(pot, stack, min_raise=2, street=1)
    env = evaluator.env_view(roots, boards.numpy())
    model = leaf_eval.ValueMLP(width=64, depth=2, dtype=torch.float32, seed=2).to(cuda_device)
    ev = evaluator.SubgameEvaluator(cuda_device, iterations=3, max_raises=2, model=model, leaf_chunk=64,
                                    generator=torch.Generator().manual_seed(1))
    ranges = torch.empty(n, 2, 1326).exponential_(generator=g)
    hit = torch.zeros(n, 52, dtype=torch.bool)
    hit.scatter_(1, boards[:, :3], True)
    c1, c2 = np.triu_indices(52, k=1)
    ranges = ranges * (~(hit[:, torch.from_numpy(c1)] | hit[:, torch.from_numpy(c2)]))[:, None, :]
    ranges = ranges / ranges.sum(-1, keepdim=True)
    ev.initialize_subgame(env, torch.arange(n), ranges)
    assert ev.layout.num_model_leaves > 0
    nxt = ev.evaluate_cfr()
    assert (nxt.state.street == 2).all() or len(nxt.nodes) == 0 or (nxt.state.street >= 1).all()
    value_batch, pre_batch, policy_batch = ev.training_data()
    assert len(value_batch) == n and len(pre_batch) == n
    assert np.array_equal(pre_batch.statistics["street"].cpu().numpy(), np.zeros(n, dtype=np.int64))
    assert (pre_batch.statistics["board"].cpu().numpy() == -1).all()  # no board before the flop
    for t in (value_batch.value_targets, pre_batch.value_targets, policy_batch.policy_targets):
        assert torch.isfinite(t).all()
    # against the CPU oracle running the same network (fp32 GEMMs in another summation order, three
    # iterations of amplification: 1e-3; the solver alone is held to 1e-5 in test_gpu_leaf_eval.py)
    from oracle import cfr as ocfr, chance as ochance

    cpu_model = leaf_eval.ValueMLP(width=64, depth=2, dtype=torch.float32, seed=2)
    trees = ev.trees
    root_of = torch.from_numpy(trees.root_of)

    def leaf_fn(beliefs, idx):
        ctx = leaf_eval.leaf_context(trees, idx.numpy())
        return ochance.single_card_chance_values(
            beliefs, boards[root_of[idx]], lambda post, samples, lookup: cpu_model(post, samples, ctx[lookup]))

    o = ocfr.SubgameOracle(trees.oracle_dict(boards.numpy()), ranges, iterations=3, leaf_fn=leaf_fn).solve()
    torch.testing.assert_close(value_batch.value_targets.cpu(), o.values_avg[:n].clamp(-1, 1), rtol=1e-3, atol=1e-5)
    top = trees.depth_offsets[-2]
    A = trees.num_actions
    by_src = torch.zeros(top, A, 1326)
    by_src[torch.from_numpy(trees.parent_index[n:]), torch.from_numpy(trees.action_from_parent[n:])] = o.policy_avg[n:]
    keep = torch.from_numpy(~trees.leaf_mask[:top])
    torch.testing.assert_close(policy_batch.policy_targets.cpu(), by_src.permute(0, 2, 1)[keep], rtol=1e-3, atol=1e-4)


def test_start_policy_from_a_belief_dependent_policy_head(cuda_device, golden_dir):
    """`initialize_policy_and_beliefs` upstream asks the policy head level by level, because a level's beliefs
    follow from the policies above it.  With a head whose logits read the beliefs: the start policy equals the
    upstream one, and the solve that follows (warm start of type `model`) matches too."""
    import os

    from poker2_b200 import evaluator as pev, tree as ptree

    z = np.load(os.path.join(golden_dir, "cfr_policy_head.npz"))
    n = z["boards"].shape[0]
    roots = ptree.root_states(z["pot"], z["stack"], min_raise=2)
    ev = pev.SubgameEvaluator(cuda_device, iterations=int(z["iterations"]), max_depth=int(z["max_depth"]),
                              max_raises=int(z["cap"]), warm_start_iterations=int(z["warm_start_iterations"]),
                              warm_start_multiplier=float(z["warm_start_multiplier"]),
                              generator=torch.Generator().manual_seed(5))
    env = pev.env_view(roots, z["boards"].astype(np.int64))
    ev.initialize_subgame(env, torch.arange(n), torch.from_numpy(z["ranges"]))
    assert ev.trees.total_nodes == int(z["total_nodes"])
    A = ev.trees.num_actions
    fixed = torch.randn(1326, A, generator=torch.Generator().manual_seed(31))
    w = torch.linspace(-1.0, 1.0, A)
    to_act = torch.from_numpy(ev.trees.state.to_act).long()

    def head(nodes, beliefs):
        mine = beliefs.cpu().gather(1, to_act[nodes][:, None, None].expand(-1, 1, 1326)).squeeze(1)
        return fixed[None] + 30.0 * mine[:, :, None] * w[None, None, :]

    start = ev.start_policy_from_head(head)
    torch.testing.assert_close(start.cpu()[n:], torch.from_numpy(z["start_policy"])[n:], rtol=1e-5, atol=1e-6)
    # the solve that follows: from the helper's policy (its 1e-7 differences from the upstream start policy
    # grow through the warm start's seeding and eight iterations of regret matching: 2e-3), and from the
    # upstream start policy itself (the solver's usual tolerance)
    ev.evaluate_cfr(start_policy=start.cpu())
    res = ev._result
    torch.testing.assert_close(res.level_major(res.policy_avg).cpu()[n:], torch.from_numpy(z["policy_avg"])[n:],
                               rtol=2e-3, atol=5e-4)
    torch.testing.assert_close(res.root_values[..., :1326].cpu(), torch.from_numpy(z["root_values"]), rtol=2e-3, atol=5e-4)
    ev.evaluate_cfr(start_policy=torch.from_numpy(z["start_policy"]))
    res = ev._result
    torch.testing.assert_close(res.level_major(res.policy_avg).cpu()[n:], torch.from_numpy(z["policy_avg"])[n:],
                               rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(res.root_values[..., :1326].cpu(), torch.from_numpy(z["root_values"]), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(res.exploitability.cpu(), torch.from_numpy(z["exploitability"]), rtol=1e-4, atol=1e-6)

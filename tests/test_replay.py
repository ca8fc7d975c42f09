"""The device-resident replay ring against the upstream `RebelReplayBuffer` fed the same seeded
batches with the same generator seed (tests/golden/golden_replay.py)."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))


def test_replay_ring_matches_upstream_buffer(golden_dir):
    from golden_replay import SIZES, seeded_batch  # plain-tensor batch builder shared with the generator

    from poker2_b200 import replay
    from poker2_b200.upstream_adapter import FeatureView, RebelBatchLike

    z = np.load(os.path.join(golden_dir, "replay.npz"))
    assert z["sizes"].tolist() == SIZES
    buf = replay.ReplayRing(12, 5, 2, 4, "cpu", policy_targets=False, decimate=0.5,
                            generator=torch.Generator().manual_seed(77))
    for k, n in enumerate(SIZES):
        b = seeded_batch(n, 100 + k)
        buf.add_batch(RebelBatchLike(FeatureView(b["context"], b["street"], b["to_act"], b["board"], b["beliefs"]),
                                     b["legal"], value_targets=b["values"], statistics={"pot": b["pot"]}))
    uniform = buf.sample(6)
    strat = buf.sample(5, stratify_streets=[0.1, 0.2, 0.3, 0.4])
    assert (buf.position, buf.size, len(buf)) == (int(z["position"]), int(z["size"]), int(z["size"]))
    assert np.array_equal(buf.features.context.numpy(), z["context"])
    assert np.array_equal(buf.features.street.numpy(), z["street"])
    assert np.array_equal(buf.features.board.numpy(), z["board"])
    assert np.array_equal(buf.features.beliefs.sum(dim=1).numpy(), z["beliefs_sum"])
    assert np.array_equal(buf.value_targets.sum(dim=(1, 2)).numpy(), z["values_sum"])
    assert np.array_equal(buf.legal_masks.numpy(), z["legal"])
    assert np.array_equal(buf.statistics["pot"].numpy(), z["pot"])
    assert np.array_equal(buf.sample_count.numpy(), z["sample_count"])
    assert np.array_equal(uniform.statistics["pot"].numpy(), z["uniform_pot"])
    assert np.array_equal(strat.statistics["pot"].numpy(), z["strat_pot"])
    assert np.array_equal(strat.features.street.numpy(), z["strat_street"])
    buf.clear()
    assert len(buf) == 0


def test_dense_evaluator_keyword_constructor_maps_to_the_solver_settings():
    """`B200CFREvaluator.from_keywords` takes the arguments of the dense `RebelCFREvaluator`
    (rebel_cfr_evaluator.py:73-100) with its defaults: linear CFR with the CFR+ clamp, cfr_avg, a `model_br`
    warm start of 15 iterations and running value targets."""
    from types import SimpleNamespace

    import torch

    from poker2_b200.upstream_adapter import B200CFREvaluator

    ev = B200CFREvaluator.from_keywords(8, SimpleNamespace(sb=5, bb=10), None, [0.5, 1.0], 4, 40, torch.device("cpu"),
                                        torch.float32, torch.Generator().manual_seed(0))
    inner = ev._ev
    assert ev.root_nodes == 8 and ev.cfr_iterations == 40 and ev.num_actions == 5 and ev.num_players == 2
    assert (inner.cfr_type, inner.cfr_plus, inner.cfr_avg, inner.running_values) == ("linear", True, True, True)
    assert (inner.warm_start_iterations, inner.warm_start_type, inner.warm_start_multiplier) == (15, "model_br", 1.0)
    assert (inner.bb, inner.max_depth, inner.sample_epsilon) == (10, 4, 0.25)
    ev = B200CFREvaluator.from_keywords(2, SimpleNamespace(bb=2), None, [1.0], 3, 12, "cpu", warm_start_iterations=0,
                                        cfr_type="discounted_plus", cfr_avg=False, cfr_plus=False, dcfr_alpha=2.0,
                                        dcfr_alpha_final=4.0, dcfr_delay=5, value_targets_from_final_policy=True,
                                        policy_delta_stats=True)
    inner = ev._ev
    assert (inner.cfr_type, inner.alpha, inner.alpha_final, inner.dcfr_delay) == ("discounted_plus", 2.0, 4.0, 5)
    assert not inner.running_values and not inner.cfr_avg and inner.policy_delta_stats and ev.num_actions == 4

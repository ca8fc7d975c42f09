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

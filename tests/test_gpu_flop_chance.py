"""Flop chance values on the GPU against the upstream helper's outputs and the host tables
against the upstream tables."""
import os

import numpy as np
import pytest
import torch


def test_flop_tables_match_upstream(golden_dir):
    from poker2_b200 import flop_chance

    z = np.load(os.path.join(golden_dir, "flop_chance.npz"))
    cards, counts = flop_chance.canonical_flops()
    assert np.array_equal(cards, z["canonical"]) and np.array_equal(counts, z["counts"])
    assert np.array_equal(flop_chance.combo_perm_table(), z["combo_perm"].astype(np.int32))
    assert int(counts.sum()) == 22100


@pytest.mark.gpu
def test_flop_chance_values_match_upstream(cuda_device, golden_dir):
    from poker2_b200 import flop_chance

    z = np.load(os.path.join(golden_dir, "flop_chance.npz"))
    cw = torch.from_numpy(z["card_w"]).to(cuda_device)
    hw = torch.from_numpy(z["hand_w"]).to(cuda_device)

    def fn(post, boards, root):
        scale = cw[boards[:, :3]].sum(dim=1).view(-1, 1, 1)
        return torch.stack([post[:, 1], -post[:, 0]], dim=1) * scale + hw.view(1, 1, -1) * 0.125

    bel = torch.from_numpy(z["beliefs"]).to(cuda_device)
    sampled = flop_chance.flop_chance_values(bel, fn, torch.Generator().manual_seed(int(z["sampled_seed"])))
    torch.testing.assert_close(sampled.cpu(), torch.from_numpy(z["sampled"]), rtol=1e-5, atol=1e-6)
    exhaustive = flop_chance.flop_chance_values(bel, fn, None, sample_size=0, num_perm_samples=0)
    torch.testing.assert_close(exhaustive.cpu(), torch.from_numpy(z["exhaustive"]), rtol=1e-5, atol=1e-6)

"""Turn subgames with leaves valued by an MLP averaged over the river card (the chance
helper as leaf evaluator) against the CPU oracle running the same network."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(n, seed):
    g = torch.Generator().manual_seed(seed)
    boards = torch.stack([torch.randperm(52, generator=g)[:4] for _ in range(n)])
    ranges = torch.empty(n, 2, 1326).exponential_(generator=g)
    from oracle import cards

    allowed = torch.from_numpy(cards.allowed_mask(boards.numpy()))
    ranges = ranges * allowed[:, None, :]
    ranges = ranges / ranges.sum(-1, keepdim=True)
    pot = torch.randint(20, 201, (n,), generator=g)
    stack = torch.randint(100, 1001, (n,), generator=g)
    return boards, ranges, pot, stack


def test_turn_subgames_with_chance_averaged_mlp_leaves(cuda_device):
    from oracle import cfr as ocfr, chance as ochance
    from poker2_b200 import leaf_eval, solver

    n, iterations = 3, 6
    boards, ranges, pot, stack = _inputs(n, 21)
    model = leaf_eval.ValueMLP(width=64, depth=2, dtype=torch.float32, seed=3)
    res, trees, sv = solver.solve_subgames_with_model(
        boards, ranges, pot, stack, model.to(cuda_device), street=2, iterations=iterations, max_raises=2,
        device=cuda_device, chunk=16)
    layout = sv.layout
    assert layout.num_model_leaves > 0 and sv.launches == 2 * (iterations + 2)

    # the oracle with the same network on the CPU
    cpu_model = leaf_eval.ValueMLP(width=64, depth=2, dtype=torch.float32, seed=3)
    boards5 = np.concatenate([boards.numpy(), np.full((n, 1), -1)], axis=1)
    root_of = torch.from_numpy(trees.root_of)

    def leaf_fn(beliefs, idx):
        ctx = leaf_eval.leaf_context(trees, idx.numpy())
        lb = torch.from_numpy(boards5)[root_of[idx]]
        return ochance.single_card_chance_values(
            beliefs, lb, lambda post, samples, lookup: cpu_model(post, samples, ctx[lookup]))

    o = ocfr.SubgameOracle(trees.oracle_dict(boards5), ranges, iterations=iterations, leaf_fn=leaf_fn).solve()
    got_pol = res.level_major(res.policy_avg).cpu()[n:]
    got_val = res.root_values[..., :1326].cpu()
    # the network's GEMMs run in different summation orders on the two devices, and the
    # iterations amplify the difference: 1e-3 relative after 6 iterations
    torch.testing.assert_close(got_val, o.values_avg[:n], rtol=1e-3, atol=1e-5)
    torch.testing.assert_close(got_pol, o.policy_avg[n:], rtol=1e-3, atol=1e-4)


def test_fused_bf16_leaf_pipeline_equals_generic_path(cuda_device):
    """The fused expansion (network input rows written directly in bf16) and the bf16 mean give
    the bits of expand_next_card -> cast -> network -> cast -> indexed mean."""
    from poker2_b200 import leaf_eval

    g = torch.Generator().manual_seed(5)
    L = 37
    boards = torch.full((L, 5), -1, dtype=torch.int64)
    for i in range(L):
        boards[i, :4] = torch.randperm(52, generator=g)[:4]
    bel = torch.zeros(L, 2, 1344)
    bel[..., :1326] = torch.empty(L, 2, 1326).exponential_(generator=g)
    bel[3, 1] = 0  # an empty range: uniform fallback over the allowed combos
    bel = (bel / bel.sum(-1, keepdim=True).clamp(min=1e-30)).to(cuda_device)
    ctx = torch.rand(L, 3, generator=g)
    model = leaf_eval.ValueMLP(width=128, depth=2, dtype=torch.bfloat16, seed=1).to(cuda_device)
    fused = leaf_eval.ChanceLeafEvaluator(model, boards, ctx, cuda_device, chunk=16)
    assert fused.fused
    generic = leaf_eval.ChanceLeafEvaluator(model, boards, ctx, cuda_device, chunk=16)
    generic.fused = False
    a = fused(bel)
    b = generic(bel)
    assert a.shape == (L, 2, 1344) and b.shape == (L, 2, 1326)
    assert torch.equal(a[..., :1326], b)

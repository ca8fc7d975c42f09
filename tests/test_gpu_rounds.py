"""Two consecutive rounds of the data-generation loop through the upstream-shaped evaluator
(`upstream_adapter.B200CFREvaluator`): the environment the first round hands to the second, the
statistics of both rounds and the training batches of the second, against a trace of the upstream
evaluator run with the same generator seeds (tests/golden/golden_rounds.py)."""
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-6


def _cfg(z, num_envs):
    search = SimpleNamespace(
        depth=int(z["max_depth"]), iterations=int(z["iterations"]), warm_start_iterations=0, warm_start_type="model",
        warm_start_multiplier=1.0, cfr_type="discounted", cfr_avg=False, cfr_plus=False, dcfr_alpha=1.5, dcfr_beta=0.0,
        dcfr_gamma=2.0, dcfr_alpha_final=None, dcfr_beta_final=None, dcfr_gamma_final=None, dcfr_plus_delay=0,
        sample_epsilon=float(z["sample_epsilon"]), value_targets_from_final_policy=True)
    return SimpleNamespace(search=search, env=SimpleNamespace(bet_bins=[0.5, 1.0], sb=1, bb=2), num_envs=num_envs, seed=0)


class PotEcho:
    """The stand-in value network of the golden run (tests/golden/golden_cfr.py, PotEchoModel) in the
    call convention of this library's leaf evaluators; zero-sum enforcement on, as in that run."""

    enforce_zero_sum = True

    def __init__(self, w):
        self.w = w

    def __call__(self, beliefs, boards, context):
        sw = (0.5 + context[:, 0].clamp(0.0, 10.0)).view(-1, 1) * self.w.to(beliefs.device).view(1, 1326)
        return torch.stack([sw + beliefs[:, 1], sw * (-0.5) + beliefs[:, 0]], dim=1)


def _check_stats(stats, z, prefix):
    for key in ("cfr_entropy", "mean_positive_regret", "mean_regret_bound", "local_exploitability",
                "local_exploitability_max", "local_exploitability_min", "evaluator_street", "evaluator_total_nodes",
                "evaluator_root_nodes", "evaluator_tree_depth"):
        assert stats[key] == pytest.approx(float(z[prefix + key]), rel=1e-4, abs=1e-6), key
    for key in ("fold", "call", "bet", "allin"):
        assert stats["action_mix"][key] == pytest.approx(float(z[f"{prefix}action_mix.{key}"]), rel=1e-4, abs=1e-6), key
    for name, value in stats["local_exploitability_street"].items():
        assert value == pytest.approx(float(z[f"{prefix}local_exploitability_street.{name}"]), rel=1e-4, abs=1e-6)


def test_policy_delta_statistics_of_both_rounds(cuda_device, golden_dir):
    """`cfr_delta.*` recorded on request (the solve then runs pass by pass): turn subgames with leaves valued by
    the model in round one, river subgames in round two, against the statistics of the upstream trace."""
    from poker2_b200 import upstream_adapter as ua

    z = np.load(os.path.join(golden_dir, "rounds_turn_river.npz"))
    n = z["boards"].shape[0]
    env = SimpleNamespace(**{name: z["env0_" + name] for name in ua.ENV_FIELDS}, raises=z["env0_raises"])
    model = PotEcho(torch.from_numpy(z["hand_weights"]))
    beliefs, idx = torch.from_numpy(z["ranges"]), torch.arange(n)
    for prefix, seed in (("stats1_", "seed_round1"), ("stats2_", "seed_round2")):
        ev = ua.B200CFREvaluator(model, cuda_device, _cfg(z, idx.shape[0]), torch.Generator().manual_seed(int(z[seed])),
                                 max_raises=int(z["cap"]), policy_delta_stats=True)
        ev.initialize_subgame(env, idx, beliefs)
        pbs = ev.evaluate_cfr()
        _check_stats(ev.stats, z, prefix)
        for q in (0, 25, 50, 75, 100):
            got, want = ev.stats[f"cfr_delta.{q}"], float(z[f"{prefix}cfr_delta.{q}"])
            print(f"{prefix}cfr_delta.{q}: {got:.8f} (upstream {want:.8f})")
            assert got == pytest.approx(want, rel=1e-4, abs=1e-6)
        env, beliefs, idx = pbs.env, pbs.beliefs, torch.arange(pbs.env.N, device=cuda_device)


def test_two_rounds_match_the_upstream_loop(cuda_device, golden_dir):
    from poker2_b200 import upstream_adapter as ua

    z = np.load(os.path.join(golden_dir, "rounds_turn_river.npz"))
    n = z["boards"].shape[0]
    env0 = SimpleNamespace(**{name: z["env0_" + name] for name in ua.ENV_FIELDS}, raises=z["env0_raises"])
    model = PotEcho(torch.from_numpy(z["hand_weights"]))
    ev = ua.B200CFREvaluator(model, cuda_device, _cfg(z, n), torch.Generator().manual_seed(int(z["seed_round1"])),
                             max_raises=int(z["cap"]))
    assert ev.root_nodes == n and ev.num_players == 2 and ev.cfr_iterations == int(z["iterations"])
    ev.initialize_subgame(env0, torch.arange(n), torch.from_numpy(z["ranges"]))
    pbs = ev.evaluate_cfr()
    # the state handed to the next round: every tensor of the upstream environment at the sampled states
    assert pbs.env.N == z["env1_pot"].shape[0]
    for name in ua.ENV_FIELDS:
        got, want = getattr(pbs.env, name).cpu().numpy(), z["env1_" + name]
        if want.dtype.kind == "f":
            np.testing.assert_allclose(got, want, rtol=1e-6, err_msg=name)
        else:
            assert np.array_equal(got, want), (name, got.tolist(), want.tolist())
    torch.testing.assert_close(pbs.beliefs.cpu(), torch.from_numpy(z["beliefs1"]), rtol=RTOL, atol=ATOL)
    _check_stats(ev.stats, z, "stats1_")
    value1, _, _ = ev.training_data()
    torch.testing.assert_close(value1.value_targets.cpu(), torch.from_numpy(z["value_targets1"]), rtol=RTOL, atol=ATOL)

    # round two starts from the returned state, as rebel_data_generator.py:69-75 does
    n2 = pbs.env.N
    ev2 = ua.B200CFREvaluator(model, cuda_device, _cfg(z, n2), torch.Generator().manual_seed(int(z["seed_round2"])),
                              max_raises=int(z["cap"]))
    ev2.initialize_subgame(pbs.env, torch.arange(n2, device=cuda_device), pbs.beliefs)
    assert ev2.stats["evaluator_total_nodes"] == float(z["total_nodes2"])
    pbs2 = ev2.evaluate_cfr()
    assert pbs2.env.N == int(z["continuing2"])
    _check_stats(ev2.stats, z, "stats2_")
    value, pre, policy = ev2.training_data()
    close = lambda a, b: torch.testing.assert_close(a.cpu(), torch.from_numpy(b), rtol=RTOL, atol=ATOL)  # noqa: E731
    close(value.value_targets, z["value_targets2"])
    close(value.features.beliefs, z["value_beliefs2"])
    close(value.features.context, z["value_context2"])
    assert np.array_equal(value.features.board.cpu().numpy(), z["value_board2"])
    assert np.array_equal(value.features.to_act.cpu().numpy(), z["value_to_act2"])
    assert np.array_equal(value.legal_masks.cpu().numpy(), z["value_legal2"])
    assert np.array_equal(value.statistics["pot"].cpu().numpy(), z["value_pot2"])
    close(value.statistics["local_exploitability"], z["value_exploitability2"])
    close(pre.value_targets, z["pre_value_targets2"])
    close(pre.features.beliefs, z["pre_beliefs2"])
    assert np.array_equal(pre.features.board.cpu().numpy(), z["pre_board2"])
    assert np.array_equal(pre.statistics["street"].cpu().numpy(), z["pre_street2"])
    assert len(policy) == int(z["policy_count2"])
    rows = torch.from_numpy(z["policy_rows2"])
    close(policy.policy_targets.cpu()[rows], z["policy_targets2"])
    close(policy.features.beliefs.cpu()[rows], z["policy_beliefs2"])
    # the batch helpers the replay hand-off uses
    both = ua.RebelBatchLike.cat([value, pre])
    assert len(both) == len(value) + len(pre) and both[:2].value_targets.shape == (2, 2, 1326)
    assert both.to(torch.device("cpu")).features.board.device.type == "cpu"

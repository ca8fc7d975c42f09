"""Fused CFR kernel (through the C ABI) against golden vectors from the upstream evaluator
and against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

# fp32 strategies and values: 1e-5 relative (project brief), plus a small absolute term for
# entries that are (near) zero on one side
RTOL, ATOL = 1e-5, 1e-6


def _solve_golden(z, device, **kw):
    from poker2_b200 import solver

    cap = int(z["cap"])
    res, trees = solver.solve_subgames(
        z["boards"].astype(np.int64), torch.from_numpy(z["ranges"]), z["pot"], z["stack"],
        iterations=int(z["iterations"]), max_depth=int(z["max_depth"]), max_raises=None if cap < 0 else cap,
        device=device, **kw)
    assert trees.total_nodes == int(z["total_nodes"])
    return res, trees


def _report(name, got, want):
    err = (got - want).abs()
    rel = err / want.abs().clamp(min=1e-6)
    print(f"{name}: max abs {err.max().item():.3e}, max rel(|x|>1e-6) {rel.max().item():.3e}")


def test_short_run_all_state(cuda_device, golden_dir):
    z = np.load(os.path.join(golden_dir, "cfr_single_cap2_t8.npz"))
    res, trees = _solve_golden(z, cuda_device, keep_policy=True, keep_node_values=True)
    n = trees.num_roots
    for name, got in [("regrets", res.regrets), ("weight_sums", res.weight_sums), ("policy", res.policy),
                      ("policy_avg", res.policy_avg), ("values_avg", res.values_avg)]:
        got = res.level_major(got).cpu()
        want = torch.from_numpy(z[name])
        if name in ("regrets", "weight_sums", "policy", "policy_avg"):
            got, want = got[n:], want[n:]  # root rows carry no action
        _report(name, got, want)
        torch.testing.assert_close(got, want, rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(res.root_values[..., :1326].cpu(), torch.from_numpy(z["values_avg"][:n]),
                               rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("name", ["cfr_single_cap2_t256", "cfr_single_nocap_t32", "cfr_batch_cap2_t24"])
def test_golden_strategies_and_values(cuda_device, golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    res, trees = _solve_golden(z, cuda_device)
    n = trees.num_roots
    pol = res.level_major(res.policy_avg).cpu()[n:]
    want_pol = torch.from_numpy(z["policy_avg"])[n:]
    vals = res.root_values[..., :1326].cpu()
    want_vals = torch.from_numpy(z["root_values"])
    _report(name + " policy_avg", pol, want_pol)
    _report(name + " root_values", vals, want_vals)
    torch.testing.assert_close(pol, want_pol, rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(vals, want_vals, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("name", ["cfr_single_cap2_t8", "cfr_single_cap2_t256", "cfr_single_nocap_t32",
                                  "cfr_batch_cap2_t24"])
def test_local_exploitability_matches_upstream(cuda_device, golden_dir, name):
    """Best-response sweeps in the kernel against `_compute_exploitability` run upstream."""
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    res, _ = _solve_golden(z, cuda_device, exploitability=True)
    got, want = res.exploitability.cpu(), torch.from_numpy(z["exploitability"])
    _report(name + " exploitability", got, want)
    torch.testing.assert_close(got, want, rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(res.br_values.cpu(), torch.from_numpy(z["br_values"]), rtol=RTOL, atol=ATOL)
    # asking for exploitability must not change the solution
    torch.testing.assert_close(res.root_values[..., :1326].cpu(), torch.from_numpy(z["root_values"]),
                               rtol=RTOL, atol=ATOL)

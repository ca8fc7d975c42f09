"""The step-level kernels, composed the way the upstream fused evaluator composes its kernels
(p2/search/fused_sparse_cfr_evaluator.py:144-398), against one iteration of the upstream NON-fused
evaluator recorded method by method (tests/golden/golden_steps.py): instantaneous regrets, the
discounted update, regret matching, reach, beliefs, the average-policy mix and the value backup."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
H = 1326


@pytest.fixture(scope="module")
def S(cuda_device, golden_dir):
    from poker2_b200 import tree as ptree

    z = np.load(os.path.join(golden_dir, "steps.npz"))
    t = ptree.build_trees(ptree.root_states(z["pot"], z["stack"], min_raise=2), [0.5, 1.0], int(z["max_depth"]), bb=2,
                          max_raises=int(z["cap"]))
    assert t.total_nodes == int(z["total_nodes"])
    dev = cuda_device
    g = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    return dict(z=z, t=t, dev=dev, g=g, N=t.num_roots, M=t.total_nodes, top=t.depth_offsets[-2], offs=t.depth_offsets,
                parent=g(t.parent_index), prev_actor=g(t.prev_actor), to_act=g(t.state.to_act),
                child_count=g(t.child_count), child_offsets=g(t.child_offsets), root_of=g(t.root_of),
                allowed=g(z["allowed"]), allowed_prob=g(z["allowed_prob"]), A=t.num_actions)


def _close(name, got, want):
    """Equal bits: the step kernels round like the upstream CPU methods the fixture recorded."""
    want = torch.from_numpy(want)
    diff = (got.cpu() - want).abs().max().item()
    print(f"{name}: max abs {diff:.3e}")
    assert torch.equal(got.cpu(), want), f"{name}: max abs difference {diff:.3e}"


def _reach(S, F, policy):
    reach = torch.zeros(S["M"], 2, H, device=S["dev"])
    # root rows: 1 on the hands the board allows (the non-fused upstream code blocks every row, roots included)
    reach[: S["N"]] = S["allowed"][: S["N"], None, :].to(torch.float32)
    for d in range(len(S["offs"]) - 2):
        F.fused_reach_weights_depth_(reach, policy, S["allowed"], S["parent"], S["prev_actor"], S["offs"][d + 1],
                                     S["offs"][d + 2])
    return reach


def _beliefs(S, F, root_rows, reach):
    out = torch.zeros(S["M"], 2, H, device=S["dev"])
    out[: S["N"]] = root_rows
    F.fused_deep_beliefs_(out, out, reach, S["allowed_prob"], S["root_of"], num_roots=S["N"])
    return out


def test_regrets_and_discounted_update(S):
    from poker2_b200 import fused_cfr as F

    z, g, N, top = S["z"], S["g"], S["N"], S["top"]
    beliefs, values = g(z["before_beliefs"]), g(z["before_values"])
    src_weights = F.unblocked_mass_opp_at_parents_triton(beliefs, S["to_act"], top)
    rows = torch.arange(top, device=S["dev"])
    actor_values = values[:top][rows, S["to_act"][:top], :].contiguous()
    regrets = torch.zeros(S["M"], H, device=S["dev"])
    F.fused_regret_tail_(regrets, values, actor_values, src_weights.contiguous(), S["parent"], S["prev_actor"], bottom=N)
    _close("instantaneous regrets", regrets, z["inst_regrets"])

    class Discounted:
        name = "discounted"

    cum, ws = g(z["before_regrets"]), g(z["before_weight_sums"])
    F.fused_dcfr_update_(cum, ws, g(z["inst_regrets"]), int(z["t"]), Discounted, 1.5, 0.0, False)
    _close("cumulative regrets", cum, z["dcfr_regrets"])
    _close("weight sums", ws, z["dcfr_weight_sums"])


def test_policy_reach_beliefs_and_average_policy(S):
    from poker2_b200 import fused_cfr as F

    z, g, N, top, t = S["z"], S["g"], S["N"], S["top"], int(S["z"]["t"])
    pos = g(z["dcfr_regrets"]).clamp(min=0.0).contiguous()
    parent_sum = F.fused_parent_sum(pos, S["child_offsets"][:top].contiguous(), S["child_count"][:top].contiguous(),
                                    max_children=S["A"])
    policy = torch.zeros(S["M"], H, device=S["dev"])
    F.fused_divide_by_parent_sum_(pos[N:].contiguous(), g(z["uniform"])[N:].contiguous(), parent_sum,
                                  S["parent"][N:].contiguous(), policy[N:])
    _close("policy", policy[N:], z["after_policy_policy"][N:])
    reach = _reach(S, F, policy)
    _close("reach", reach, z["after_policy_reach"])
    root_rows = g(z["after_policy_beliefs"])[:N]
    beliefs = _beliefs(S, F, root_rows, reach)
    _close("beliefs", beliefs, z["after_policy_beliefs"])
    # average policy: reach-weighted mix (weights t^2, (t+1)^2) and renormalisation over the siblings
    avg = g(z["before_policy_avg"])
    F.fused_average_policy_mix_(avg, policy, reach, g(z["before_reach_avg"]), S["to_act"], S["parent"],
                                old=float(t ** 2.0), new=float((t + 1) ** 2.0), bottom=N)
    psum = F.fused_parent_sum(avg.contiguous(), S["child_offsets"][:top].contiguous(), S["child_count"][:top].contiguous(),
                              max_children=S["A"])
    child = avg[N:].contiguous()
    F.fused_divide_by_parent_sum_(child, child, psum, S["parent"][N:].contiguous(), avg[N:], eps=1e-5)
    avg[:N] = 0.0
    _close("policy_avg", avg, z["after_policy_policy_avg"])
    reach_avg = _reach(S, F, avg)
    _close("reach_avg", reach_avg, z["after_policy_reach_avg"])
    _close("beliefs_avg", _beliefs(S, F, g(z["after_policy_beliefs_avg"])[:N], reach_avg), z["after_policy_beliefs_avg"])


def test_block_normalize_matches_upstream_rows(S):
    from poker2_b200 import fused_cfr as F

    z, g = S["z"], S["g"]
    # un-normalised rows: root beliefs x reach; upstream blocks and normalises them (cfr_evaluator.py:254-273)
    raw = g(z["after_policy_beliefs"])[S["root_of"]][:, :, :] * 0 + g(z["after_policy_beliefs"])[: S["N"]][S["root_of"]]
    raw = (raw * g(z["after_policy_reach"])).contiguous()
    F.fused_block_and_normalize_beliefs_(raw, S["allowed"], S["allowed_prob"])
    _close("normalised beliefs", raw[S["N"]:], z["after_policy_beliefs"][S["N"]:])


def test_value_backup(S):
    from poker2_b200 import fused_cfr as F

    z, g, N, top, offs = S["z"], S["g"], S["N"], S["top"], S["offs"]
    policy, beliefs = g(z["after_policy_policy"]), g(z["after_policy_beliefs"])
    values = g(z["leaf_values"]).clone()
    idx = S["to_act"][:top, None, None].expand(-1, -1, H)
    actor_beliefs = beliefs[:top].gather(1, idx).squeeze(1)
    marginal = (actor_beliefs.index_select(0, S["parent"][N:]) * policy[N:]).contiguous()
    opp = torch.zeros_like(policy)
    opp[N:] = F.unblocked_mass_ratio_indirect_triton(marginal, actor_beliefs.contiguous(), S["parent"][N:].contiguous())
    for d in range(len(offs) - 3, -1, -1):
        a, b = offs[d], offs[d + 1]
        F.fused_weighted_parent_sum(values, S["prev_actor"], policy, opp, S["child_offsets"][a:b].contiguous(),
                                    S["child_count"][a:b].contiguous(), parent_base=a, max_children=S["A"])
    _close("expected values", values, z["after_values"])

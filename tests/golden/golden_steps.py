"""One iteration of the upstream NON-fused evaluator, method by method: the state before
`cfr_iteration(t)` and the result of every step it runs (`compute_instantaneous_regrets`
cfr_evaluator.py:1117-1165, the discounted update :1346-1368, `update_policy` :1168-1193 with
`_calculate_reach_weights` :332-361, `_propagate_all_beliefs` / `_normalize_beliefs` :254-273,
363-380 and `update_average_policy` :1195-1258, `compute_expected_values` :1049-1115).  The
step-level kernels are checked against these arrays.  Imported by make_golden.py."""
from __future__ import annotations

import numpy as np
import torch

import golden_cfr as gc
from golden_cfr import save


def gen_steps() -> None:
    n = 1
    b, r, p, s = gc.seeded_inputs(51, n, (20, 200), (100, 1000))
    iterations, cap, depth, t_rec = 6, 2, 2, 4  # one root, a shallow tree: the fixture stays small
    gc.install_raise_cap(cap)
    ev = gc.make_evaluator(n, iterations, depth=depth)
    ev.initialize_subgame(gc.river_env(b, p, s), torch.arange(n), r)
    rec = {}
    snap = lambda: dict(  # noqa: E731
        policy=ev.policy_probs.clone(), policy_avg=ev.policy_probs_avg.clone(), regrets=ev.cumulative_regrets.clone(),
        weight_sums=ev.regret_weight_sums.clone(), reach=ev.self_reach.clone(), reach_avg=ev.self_reach_avg.clone(),
        beliefs=ev.beliefs.clone(), beliefs_avg=ev.beliefs_avg.clone(), values=ev.latest_values.clone())
    orig_iter, orig_inst, orig_up, orig_avg = (ev.cfr_iteration, ev.compute_instantaneous_regrets, ev.update_policy,
                                               ev.update_average_policy)
    orig_leaf, orig_ev = ev.set_leaf_values, ev.compute_expected_values
    state = {"on": False}

    def inst(values):
        out = orig_inst(values)
        if state["on"]:
            rec["inst_regrets"] = out.clone()
        return out

    def up(t):
        if state["on"]:
            rec["after_dcfr"] = dict(regrets=ev.cumulative_regrets.clone(), weight_sums=ev.regret_weight_sums.clone())
        orig_up(t)
        if state["on"]:
            rec["after_policy"] = snap()

    def avg(t):
        if state["on"]:
            rec["before_avg"] = snap()
        orig_avg(t)
        if state["on"]:
            rec["avg_after_mix"] = ev.policy_probs_avg.clone()

    def leaf(t, beliefs=None):
        orig_leaf(t, beliefs)
        if state["on"]:
            rec["leaf_values"] = ev.latest_values.clone()

    def expected(*a, **k):
        orig_ev(*a, **k)
        if state["on"] and not a and not k:
            rec["after_values"] = ev.latest_values.clone()

    ev.compute_instantaneous_regrets, ev.update_policy, ev.update_average_policy = inst, up, avg
    ev.set_leaf_values, ev.compute_expected_values = leaf, expected

    def iteration(t):
        state["on"] = t == t_rec
        if state["on"]:
            rec["before"] = snap()
        orig_iter(t)
        state["on"] = False

    ev.cfr_iteration = iteration
    ev.generator = torch.Generator().manual_seed(3)
    ev.evaluate_cfr()
    gc.install_raise_cap(None)
    out = dict(boards=b.to(torch.int16).numpy(), ranges=r.numpy(), pot=p.numpy(), stack=s.numpy(), cap=np.int64(cap),
               max_depth=np.int64(depth), t=np.int64(t_rec), total_nodes=np.int64(ev.total_nodes),
               allowed=ev.allowed_hands.numpy(), allowed_prob=ev.allowed_hands_prob.numpy(),
               uniform=ev.uniform_policy.numpy(), inst_regrets=rec["inst_regrets"].numpy(),
               dcfr_regrets=rec["after_dcfr"]["regrets"].numpy(), dcfr_weight_sums=rec["after_dcfr"]["weight_sums"].numpy(),
               leaf_values=rec["leaf_values"].numpy(), after_values=rec["after_values"].numpy())
    keep = {"before": ("regrets", "weight_sums", "beliefs", "values", "policy_avg", "reach_avg"),
            "after_policy": ("policy", "reach", "beliefs", "policy_avg", "reach_avg", "beliefs_avg")}
    for tag, names in keep.items():
        for k in names:
            out[f"{tag}_{k}"] = rec[tag][k].numpy()
    print("steps: nodes", ev.total_nodes, "arrays", len(out))
    save("steps.npz", **out)


gc.SECTIONS.update(steps=gen_steps)

"""Step-level CFR kernels with the call signatures of the upstream module
p2/search/fused_cfr_triton.py, backed by hand-written CUDA (csrc/stepops.cu).

An evaluator written against the upstream module (`FusedSparseCFREvaluator`) can switch
with `import poker2_b200.fused_cfr as fused_cfr_triton`.  All functions operate in place on
caller-owned contiguous CUDA fp32 tensors (asserts on contiguity and shape, like upstream);
index tensors are int64.  The whole-subgame kernel (`poker2_b200.solver`) is the fast path.
"""
from __future__ import annotations

import torch

from . import _lib

NUM_HANDS = _lib.NUM_HANDS


def triton_is_available() -> bool:
    """Upstream name for "the kernel backend is present" (fused_cfr_triton.py:65)."""
    return _lib.library_available()


def _require() -> None:
    if not _lib.library_available():
        raise RuntimeError("libpoker2_b200.so is not built; run `python -m poker2_b200.build`.")


def _call(name: str, dev: torch.device, *args) -> None:
    with torch.cuda.device(dev):
        _lib.call(name, *args, _lib.stream_ptr(dev))


def _p(t):
    return _lib.ptr(t)


def _scalar(value: float, like: torch.Tensor) -> torch.Tensor:
    return torch.tensor(float(value), dtype=like.dtype, device=like.device)


def _mask_bytes(mask: torch.Tensor) -> torch.Tensor:
    assert mask.is_contiguous()
    return mask.view(torch.uint8) if mask.dtype == torch.bool else mask.to(torch.uint8)


# ---- DCFR update (fused_cfr_triton.py:123-235) -----------------------------------------
def fused_dcfr_update_with_tensors_(cumulative_regrets, regret_weight_sums, regrets, t_alpha_num, t_beta_num,
                                    t_alpha_den, t_beta_den, apply_dcfr: bool, cfr_plus: bool,
                                    positive_regrets_out=None, block_size: int = 1024) -> None:
    _require()
    scal = torch.stack([t_alpha_num.reshape(()), t_beta_num.reshape(()), t_alpha_den.reshape(()),
                        t_beta_den.reshape(())]).to(torch.float32).contiguous()
    _call("p2b_step_dcfr_update", cumulative_regrets.device, _p(regrets), _p(cumulative_regrets),
          _p(regret_weight_sums), _p(positive_regrets_out), _p(scal), cumulative_regrets.numel(), int(apply_dcfr),
          int(cfr_plus))


def fused_dcfr_update_(cumulative_regrets, regret_weight_sums, regrets, t: int, cfr_type, dcfr_alpha: float,
                       dcfr_beta: float, cfr_plus: bool, positive_regrets_out=None, block_size: int = 1024) -> None:
    _require()
    if cumulative_regrets.device.type != "cuda":
        raise ValueError("fused_dcfr_update_ requires CUDA tensors.")
    kind = getattr(cfr_type, "name", str(cfr_type))
    if kind == "linear":
        raise NotImplementedError("Linear CFR path not supported; default config uses discounted_plus.")
    assert cumulative_regrets.is_contiguous() and regret_weight_sums.is_contiguous() and regrets.is_contiguous()
    assert cumulative_regrets.shape == regret_weight_sums.shape == regrets.shape
    apply_dcfr = kind in ("discounted", "discounted_plus")
    if apply_dcfr:
        an, bn = float(t ** dcfr_alpha), float(t ** dcfr_beta)
        ad, bd = an + 1.0, bn + 1.0
    else:
        an = bn = ad = bd = 1.0
    c = cumulative_regrets
    fused_dcfr_update_with_tensors_(c, regret_weight_sums, regrets, _scalar(an, c), _scalar(bn, c), _scalar(ad, c),
                                    _scalar(bd, c), apply_dcfr, cfr_plus, positive_regrets_out)


# ---- beliefs (fused_cfr_triton.py:286-335, 2039-2092) ----------------------------------
def fused_block_and_normalize_beliefs_(target, allowed_hands, allowed_hands_prob, eps: float = 1e-5) -> None:
    _require()
    assert target.is_contiguous() and allowed_hands.is_contiguous() and allowed_hands_prob.is_contiguous()
    assert target.device.type == "cuda"
    if target.dim() == 3:
        n, p, h = target.shape
        rows, stride = n * p, p
    elif target.dim() == 2:
        n, h = target.shape
        rows, stride = n, 1
    else:
        raise ValueError(f"target must be 2D or 3D, got {target.shape}")
    assert allowed_hands.shape == (n, h) and allowed_hands_prob.shape == (n, h)
    _call("p2b_step_block_normalize", target.device, _p(target), _p(_mask_bytes(allowed_hands)),
          _p(allowed_hands_prob), rows, stride, h, float(eps))


def fused_deep_beliefs_(out, root_beliefs, reach_weights, allowed_prob, root_index, num_roots=None,
                        eps: float = 1e-5, block_h: int = 2048) -> None:
    _require()
    assert out.is_contiguous() and reach_weights.is_contiguous() and allowed_prob.is_contiguous()
    assert root_beliefs.is_contiguous() and root_index.is_contiguous()
    total, two, h = out.shape
    assert two == 2 and reach_weights.shape == out.shape and allowed_prob.shape == (total, h)
    n = num_roots if num_roots is not None else root_beliefs.shape[0]
    if total <= n:
        return
    _call("p2b_step_deep_beliefs", out.device, _p(out), _p(root_beliefs), _p(reach_weights), _p(allowed_prob),
          _p(root_index), n, total, h, float(eps))


def fused_reach_weights_depth_(reach, policy, allowed_mask, parent_index, prev_actor, start: int, end: int,
                               block_h: int = 2048) -> None:
    _require()
    assert reach.is_contiguous() and policy.is_contiguous() and allowed_mask.is_contiguous()
    assert parent_index.is_contiguous() and prev_actor.is_contiguous()
    total, two, h = reach.shape
    assert two == 2 and policy.shape == (total, h) and allowed_mask.shape == (total, h)
    if end - start <= 0:
        return
    _call("p2b_step_reach_weights", reach.device, _p(reach), _p(policy), _p(_mask_bytes(allowed_mask)),
          _p(parent_index), _p(prev_actor), start, end, h)


# ---- policy (fused_cfr_triton.py:369-399, 823-914, 1279-1398) ---------------------------
def fused_regret_matching_divide_(positive_regrets, denom, uniform_fallback, out, eps: float = 1e-8,
                                  block_size: int = 1024) -> None:
    _require()
    for t in (positive_regrets, denom, uniform_fallback, out):
        assert t.is_contiguous()
    assert positive_regrets.shape == denom.shape == uniform_fallback.shape == out.shape
    _call("p2b_step_regret_matching_divide", out.device, _p(positive_regrets), _p(denom), _p(uniform_fallback),
          _p(out), out.numel(), float(eps))


def fused_average_policy_mix_with_tensors_(policy_probs_avg, policy_probs, self_reach, self_reach_avg, to_act,
                                           parent_index, old, new, total_weight, bottom: int, eps: float = 1e-5,
                                           block_h: int = 512) -> None:
    _require()
    assert policy_probs_avg.is_contiguous() and policy_probs.is_contiguous()
    assert self_reach.is_contiguous() and self_reach_avg.is_contiguous()
    assert to_act.is_contiguous() and parent_index.is_contiguous()
    total, h = policy_probs_avg.shape
    assert policy_probs.shape == (total, h) and self_reach.shape == (total, 2, h) == self_reach_avg.shape
    _call("p2b_step_average_policy_mix", policy_probs_avg.device, _p(self_reach), _p(self_reach_avg),
          _p(policy_probs), _p(policy_probs_avg), _p(to_act), _p(parent_index), _p(old), _p(new), _p(total_weight),
          bottom, total, h, float(eps))


def fused_average_policy_mix_(policy_probs_avg, policy_probs, self_reach, self_reach_avg, to_act, parent_index,
                              old: float, new: float, bottom: int, eps: float = 1e-5, block_h: int = 512) -> None:
    a = policy_probs_avg
    fused_average_policy_mix_with_tensors_(a, policy_probs, self_reach, self_reach_avg, to_act, parent_index,
                                           _scalar(old, a), _scalar(new, a), _scalar(float(old) + float(new), a),
                                           bottom=bottom, eps=eps)


def fused_parent_sum(values, child_offsets, child_count, max_children: int = 8, block_h: int = 512):
    _require()
    assert values.is_contiguous() and values.dim() == 2
    assert child_offsets.is_contiguous() and child_count.is_contiguous() and child_offsets.shape == child_count.shape
    num_parents, h = child_offsets.shape[0], values.shape[1]
    out = torch.empty(num_parents, h, device=values.device, dtype=values.dtype)
    _call("p2b_step_parent_sum", values.device, _p(values), _p(child_offsets), _p(child_count), _p(out), num_parents,
          h, 0, 0)
    return out


def fused_sibling_sum(values, child_offsets, child_count, bottom: int, num_children: int, max_children: int = 8,
                      block_h: int = 512):
    _require()
    assert values.is_contiguous() and values.dim() == 2
    assert child_offsets.is_contiguous() and child_count.is_contiguous()
    h = values.shape[1]
    out = torch.empty(num_children, h, device=values.device, dtype=values.dtype)
    _call("p2b_step_parent_sum", values.device, _p(values), _p(child_offsets), _p(child_count), _p(out),
          child_offsets.shape[0], h, 1, bottom)
    return out


def fused_divide_by_parent_sum_(pos, fallback, parent_sum, parent_index, out, eps: float = 1e-8, block_c: int = 32,
                                block_h: int = 128) -> None:
    _require()
    for t in (pos, fallback, parent_sum, parent_index, out):
        assert t.is_contiguous()
    num_children, h = pos.shape
    assert fallback.shape == pos.shape == out.shape and parent_index.shape == (num_children,)
    _call("p2b_step_divide_by_parent_sum", out.device, _p(pos), _p(fallback), _p(parent_sum), _p(parent_index),
          _p(out), num_children, h, float(eps))


# ---- values (fused_cfr_triton.py:438-668, 712-766, 1633-1889) ---------------------------
def fused_weight_child_values(values_src, prev_actor, policy_hero, policy_opp, out, block_h: int = 512) -> None:
    _require()
    assert values_src.is_contiguous() and values_src.dim() == 3 and out.is_contiguous()
    assert out.shape == values_src.shape and prev_actor.is_contiguous() and prev_actor.dim() == 1
    assert policy_hero.is_contiguous() and policy_opp.is_contiguous()
    m, p, h = values_src.shape
    assert p == 2, "Only supports 2 players."
    assert prev_actor.shape[0] == m and policy_hero.shape == (m, h) and policy_opp.shape == (m, h)
    _call("p2b_step_weight_child_values", out.device, _p(values_src), _p(prev_actor), _p(policy_hero),
          _p(policy_opp), _p(out), m, h)


def fused_update_average_values_with_tensors_(values_avg, latest_values, old, new, inv_total,
                                              block_size: int = 1024) -> None:
    _require()
    _call("p2b_step_update_average_values", values_avg.device, _p(values_avg), _p(latest_values), _p(old), _p(new),
          _p(inv_total), values_avg.numel())


def fused_update_average_values_(values_avg, latest_values, old: float, new: float, block_size: int = 1024) -> None:
    assert values_avg.is_contiguous() and latest_values.is_contiguous() and values_avg.shape == latest_values.shape
    total = float(old) + float(new)
    assert total != 0.0
    v = values_avg
    fused_update_average_values_with_tensors_(v, latest_values, _scalar(old, v), _scalar(new, v),
                                              _scalar(1.0 / total, v))


def fused_avg_values_zero_sum_(values_avg, latest_values, beliefs, old, new, inv_total, enforce_zero_sum: bool,
                               ignore_mask=None, block_h: int = 2048) -> None:
    _require()
    assert values_avg.is_contiguous() and latest_values.is_contiguous() and beliefs.is_contiguous()
    assert values_avg.shape == latest_values.shape == beliefs.shape
    assert values_avg.dim() == 3 and values_avg.shape[1] == 2
    rows, _, h = values_avg.shape
    ig = None
    if ignore_mask is not None:
        assert ignore_mask.is_contiguous() and ignore_mask.shape == (rows,)
        ig = _mask_bytes(ignore_mask)
    _call("p2b_step_mix_zero_sum", values_avg.device, _p(values_avg), _p(latest_values), _p(beliefs), _p(ig), _p(old),
          _p(new), _p(inv_total), _p(values_avg), rows, h, 0, int(enforce_zero_sum))


def fused_regret_tail_(regrets, values_achieved, actor_values, src_weights, parent_index, prev_actor, bottom: int,
                       block_h: int = 512) -> None:
    _require()
    assert regrets.is_contiguous() and regrets.dim() == 2
    assert values_achieved.is_contiguous() and values_achieved.dim() == 3 and values_achieved.shape[1] == 2
    assert actor_values.is_contiguous() and src_weights.is_contiguous() and actor_values.shape == src_weights.shape
    assert parent_index.is_contiguous() and prev_actor.is_contiguous()
    total, h = regrets.shape
    assert values_achieved.shape == (total, 2, h) and parent_index.shape == (total,) == prev_actor.shape
    _call("p2b_step_regret_tail", regrets.device, _p(values_achieved), _p(actor_values), _p(src_weights),
          _p(parent_index), _p(prev_actor), _p(regrets), bottom, total, h)


def fused_model_values_mix_with_tensors(hand_values, last_model_values, old_plus_new_over_new, old_over_new, out,
                                        block_size: int = 1024) -> None:
    _require()
    assert hand_values.is_contiguous() and last_model_values.is_contiguous() and out.is_contiguous()
    _call("p2b_step_scaled_difference", out.device, _p(hand_values), _p(last_model_values), _p(old_plus_new_over_new),
          _p(old_over_new), _p(out), hand_values.numel())


def fused_model_values_mix(hand_values, last_model_values, old: float, new: float, block_size: int = 1024):
    out = torch.empty_like(hand_values)
    fused_model_values_mix_with_tensors(hand_values, last_model_values,
                                        _scalar((old + new) / new, hand_values), _scalar(old / new, hand_values), out)
    return out


def fused_model_values_mix_zero_sum(hand_values, last_model_values, beliefs, old_plus_new_over_new, old_over_new, out,
                                    enforce_zero_sum: bool, block_h: int = 2048) -> None:
    _require()
    for t in (hand_values, last_model_values, beliefs, out):
        assert t.is_contiguous()
    assert hand_values.shape == last_model_values.shape == beliefs.shape == out.shape
    m, two, h = hand_values.shape
    assert two == 2
    _call("p2b_step_mix_zero_sum", out.device, _p(hand_values), _p(last_model_values), _p(beliefs), None,
          _p(old_plus_new_over_new), _p(old_over_new), None, _p(out), m, h, 1, int(enforce_zero_sum))


def mix_zero_sum(a, b, beliefs, coef_a, coef_b, out, mode: int = 1) -> None:
    """out = a*coef_a - b*coef_b, minus 0.5 * sum over players and hands of out * beliefs (rows of [2,H]).
    mode 1: the sum in fp64; mode 2 (H = 1326): fp32 sums in the order of the CPU row reduction, which
    reproduces `_maybe_enforce_zero_sum` of the non-fused upstream evaluator (cfr_evaluator.py:957-980) bit
    for bit."""
    _require()
    for t in (a, b, beliefs, out):
        assert t.is_contiguous()
    assert a.shape == b.shape == beliefs.shape == out.shape and a.shape[1] == 2
    m, _, h = a.shape
    _call("p2b_step_mix_zero_sum", out.device, _p(a), _p(b), _p(beliefs), None, _p(coef_a), _p(coef_b), None, _p(out),
          m, h, 1, int(mode))


def mix_zero_sum_rows(a, b, beliefs, ignore, coef_a, coef_b, scale, out, *, divide: bool = False, mode: int = 1) -> None:
    """out = (a*coef_a + b*coef_b) * scale (or / scale with `divide`), minus the zero-sum shift of rows of [2,H]
    whose `ignore` byte is 0 (mode 0: no shift, 1: fp64 sum, 2: fp32 sums in the CPU row-reduction order; H may be
    padded beyond 1326 only in modes 0 and 1).  The non-fused `update_average_values` upstream
    (cfr_evaluator.py:1260-1274) is divide=True, mode=2."""
    _require()
    for t in (a, b, beliefs, out):
        assert t.is_contiguous() and t.shape == a.shape
    m, two, h = a.shape
    assert two == 2 and (ignore is None or (ignore.is_contiguous() and ignore.shape == (m,)))
    _call("p2b_step_mix_zero_sum", out.device, _p(a), _p(b), _p(beliefs), _p(ignore), _p(coef_a), _p(coef_b), _p(scale),
          _p(out), m, h, 2 if divide else 0, int(mode))


def fused_weighted_parent_sum(values, prev_actor, policy_hero, policy_opp, child_offsets, child_count,
                              parent_base: int, max_children: int = 8, block_h: int = 2048) -> None:
    _require()
    assert values.is_contiguous() and values.dim() == 3 and values.shape[1] == 2
    for t in (prev_actor, policy_hero, policy_opp, child_offsets, child_count):
        assert t.is_contiguous()
    total, _, h = values.shape
    assert policy_hero.shape == (total, h) == policy_opp.shape and prev_actor.shape == (total,)
    _call("p2b_step_weighted_parent_sum", values.device, _p(values), _p(prev_actor), _p(policy_hero), _p(policy_opp),
          _p(child_offsets), _p(child_count), parent_base, child_offsets.shape[0], h)


# ---- unblocked mass (fused_cfr_triton.py:1029-1157, 1499-1602) --------------------------
def unblocked_mass_triton(target: torch.Tensor) -> torch.Tensor:
    _require()
    if target.device.type != "cuda":
        raise ValueError("unblocked_mass_triton requires CUDA tensors.")
    assert target.shape[-1] == NUM_HANDS, f"last dim must be {NUM_HANDS}, got {tuple(target.shape)}"
    flat = target.reshape(-1, NUM_HANDS).contiguous()
    out = torch.empty_like(flat)
    _call("p2b_step_unblocked_mass", flat.device, _p(flat), None, _p(out), flat.shape[0])
    return out.view(target.shape)


class ParentBeliefUnblockedStats:
    """Upstream caches (S, card sums) of `beliefs[:top]` here (fused_cfr_triton.py:1029-1064);
    the CUDA kernels recompute them in shared memory, so this only keeps the tensor."""

    def __init__(self, beliefs_parents: torch.Tensor) -> None:
        self.top = beliefs_parents.shape[0]
        self.beliefs_parents = beliefs_parents


def unblocked_mass_opp_at_parents_triton(beliefs, to_act, top: int, cached_stats=None) -> torch.Tensor:
    _require()
    assert beliefs.is_contiguous() and beliefs.dim() == 3 and beliefs.shape[1] == 2
    assert beliefs.shape[2] == NUM_HANDS
    rows = torch.arange(top, device=beliefs.device, dtype=torch.int64) * 2 + (1 - to_act[:top].to(torch.int64))
    out = torch.empty(top, NUM_HANDS, device=beliefs.device, dtype=beliefs.dtype)
    _call("p2b_step_unblocked_mass", beliefs.device, _p(beliefs), _p(rows.contiguous()), _p(out), top)
    return out


def unblocked_mass_ratio_indirect_triton(numer_target, denom_target, parent_index, eps: float = 1e-5,
                                         denom_stats=None) -> torch.Tensor:
    _require()
    assert numer_target.is_contiguous() and denom_target.is_contiguous() and parent_index.is_contiguous()
    assert numer_target.shape[1] == NUM_HANDS == denom_target.shape[1]
    out = torch.empty_like(numer_target)
    _call("p2b_step_unblocked_mass_ratio", out.device, _p(numer_target), _p(denom_target), _p(parent_index), _p(out),
          numer_target.shape[0], float(eps))
    return out


def unblocked_mass_ratio_triton(numer_target, denom_target, eps: float = 1e-5) -> torch.Tensor:
    _require()
    assert numer_target.shape == denom_target.shape and numer_target.shape[-1] == NUM_HANDS
    n = numer_target.reshape(-1, NUM_HANDS).contiguous()
    d = denom_target.reshape(-1, NUM_HANDS).contiguous()
    out = torch.empty_like(n)
    _call("p2b_step_unblocked_mass_ratio", out.device, _p(n), _p(d), None, _p(out), n.shape[0], float(eps))
    return out.view(numer_target.shape)


# ---- iteration scalars (fused_cfr_triton.py:2100-2158) ----------------------------------
class TScalars:
    """0-D device tensors holding the scalars that depend on the iteration number; fill
    them on the host with `update` before launching (or replaying) the step kernels."""

    def __init__(self, device: torch.device, dtype: torch.dtype = torch.float32) -> None:
        z = lambda: torch.zeros((), dtype=dtype, device=device)  # noqa: E731
        self.device, self.dtype = device, dtype
        self.t_alpha_num, self.t_beta_num, self.t_alpha_den, self.t_beta_den = z(), z(), z(), z()
        self.mix_old, self.mix_new, self.mix_total, self.mix_inv_total = z(), z(), z(), z()
        self.mix_onon, self.mix_oon = z(), z()
        self.t_tensor = torch.zeros((), dtype=torch.long, device=device)

    def update(self, t: int, dcfr_alpha: float, dcfr_beta: float, mix_old: float, mix_new: float) -> None:
        an, bn = float(t ** dcfr_alpha), float(t ** dcfr_beta)
        self.t_alpha_num.fill_(an)
        self.t_beta_num.fill_(bn)
        self.t_alpha_den.fill_(an + 1.0)
        self.t_beta_den.fill_(bn + 1.0)
        total = float(mix_old) + float(mix_new)
        self.mix_old.fill_(float(mix_old))
        self.mix_new.fill_(float(mix_new))
        self.mix_total.fill_(total)
        self.mix_inv_total.fill_(1.0 / total if total != 0.0 else 1.0)
        if float(mix_new) != 0.0:
            self.mix_onon.fill_(total / float(mix_new))
            self.mix_oon.fill_(float(mix_old) / float(mix_new))
        self.t_tensor.fill_(int(t))


# ---- showdown EV from strength-sorted inputs (fused_cfr_triton.py:2271-2320) --------------
def showdown_ev_triton(b_opp_sorted: torch.Tensor, c1_sorted: torch.Tensor, c2_sorted: torch.Tensor,
                       L_idx: torch.Tensor, R_idx: torch.Tensor, eps: float = 1e-8, block_k: int = 32,
                       block_j: int = 128) -> torch.Tensor:
    """`EV_hand_sorted` [M,H] from sorted-order inputs: b_opp_sorted [M,H] fp32 (the opponent's normalised
    beliefs in strength order, zero on the hands that use a board card), c1_sorted / c2_sorted [M,H] the
    hole cards of every sorted position, L_idx / R_idx [M,H] its tie group [L,R).  As upstream, the caller
    permutes the result back, multiplies by the hand mask and scales by potential / scale.  block_k and
    block_j tune the upstream kernel's tiles and are accepted for the signature only: one thread block
    handles a row with one prefix over the positions and one per card."""
    _require()
    if b_opp_sorted.device.type != "cuda":
        raise ValueError("showdown_ev_triton requires CUDA tensors.")
    assert b_opp_sorted.is_contiguous() and b_opp_sorted.dim() == 2 and b_opp_sorted.dtype == torch.float32
    M, H = b_opp_sorted.shape
    assert c1_sorted.shape == (M, H) and c2_sorted.shape == (M, H)
    assert L_idx.shape == (M, H) and R_idx.shape == (M, H)
    c1, c2, lo, hi = (x.to(torch.int32).contiguous() for x in (c1_sorted, c2_sorted, L_idx, R_idx))
    out = torch.empty(M, H, device=b_opp_sorted.device, dtype=torch.float32)
    _call("p2b_showdown_ev_sorted", out.device, _p(b_opp_sorted), _p(c1), _p(c2), _p(lo), _p(hi), M, H, float(eps), _p(out))
    return out


# ---- CUDA graph capture of a whole cfr_iteration (fused_cfr_triton.py:2322-2457) ---------
class _EvaluatorStateSnapshot:
    """Copies of the evaluator tensors an iteration changes; `restore_to` puts them back."""

    NAMES = ("policy_probs", "policy_probs_avg", "policy_probs_sample", "cumulative_regrets", "regret_weight_sums",
             "self_reach", "self_reach_avg", "beliefs", "beliefs_avg", "latest_values", "values_avg")

    def __init__(self, names, tensors):
        self.names, self.tensors = tuple(names), tuple(tensors)

    @classmethod
    def from_evaluator(cls, evaluator) -> "_EvaluatorStateSnapshot":
        names = [n for n in cls.NAMES if isinstance(getattr(evaluator, n, None), torch.Tensor)]
        return cls(names, [getattr(evaluator, n).detach().clone() for n in names])

    def restore_to(self, evaluator) -> None:
        for name, saved in zip(self.names, self.tensors):
            getattr(evaluator, name).copy_(saved)

    def max_abs_diff(self, other: "_EvaluatorStateSnapshot") -> dict:
        assert self.names == other.names
        return {n: (a - b).abs().max().item() for n, a, b in zip(self.names, self.tensors, other.tensors)}


class GraphedCFRIteration:
    """Captures `evaluator.cfr_iteration` in a CUDA graph and replays it for other iterations, with the
    interface of upstream's class: `capture(t_capture, num_warmup)` runs real warm-up iterations (they move
    the evaluator's state, as upstream's do), then records one iteration; `replay(t)` refreshes the device
    scalars through `evaluator.prepare_replay(t)` outside the graph and launches it.  The evaluator must
    keep its iteration scalars on the device and honour `_skip_t_scalars_update`
    (`step_evaluator.StepCFREvaluator` does).  Replayed iterations must take the Python branches of the
    captured one (both past the average-policy delay, for one), and the trees are baked in."""

    def __init__(self, evaluator) -> None:
        if evaluator.device.type != "cuda":
            raise ValueError("GraphedCFRIteration requires a CUDA evaluator.")
        self.evaluator = evaluator
        self._graph = None
        self._captured_t = None

    def capture(self, t_capture: int, num_warmup: int = 2) -> None:
        ev = self.evaluator
        if not hasattr(ev, "_t_scalars"):
            raise ValueError("Evaluator must keep its iteration scalars on the device (a ._t_scalars TScalars holder) "
                             "for graph capture.")
        for i in range(num_warmup):
            ev.cfr_iteration(t_capture + i)
        ev.prepare_replay(t_capture)
        prev_skip = ev._skip_t_scalars_update
        ev._skip_t_scalars_update = True
        try:
            with torch.cuda.device(ev.device):
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    ev.cfr_iteration(t_capture)  # one run on the capture stream, scalars already filled
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    ev.cfr_iteration(t_capture)
        finally:
            ev._skip_t_scalars_update = prev_skip
        self._graph, self._captured_t = graph, int(t_capture)

    def replay(self, t: int | None = None) -> None:
        if self._graph is None:
            raise RuntimeError("capture() must be called before replay().")
        if t is not None:
            self.evaluator.prepare_replay(t)
        self._graph.replay()

    @property
    def captured_t(self):
        return self._captured_t

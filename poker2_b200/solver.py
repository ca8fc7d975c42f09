"""Batched subgame solving on the GPU: host-side preparation and the call into the fused
CFR kernel (`p2b_cfr_solve`).

`solve_subgames` does, for a batch of independent river subgames, what the upstream
`initialize_subgame` + `evaluate_cfr` do (p2/search/cfr_evaluator.py:770-828, 1497-1528,
with `value_targets_from_final_policy`), and returns the arrays `training_data` reads
(:1384-1495): average policy per node, values of the average policy at the roots, plus the
cumulative regrets and weight sums.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from . import _lib, tree as ptree
from .showdown import BoardTables

HPAD = 1344
NUM_HANDS = 1326
MAX_NODES = 320  # nodes of one subgame (general kernel); the lean iteration kernel takes those of up to 160
MAX_CHILDREN = 8  # actions per node (general kernel); batches of up to 6 run their iteration passes in the lean kernel

NODE_DTYPE = np.dtype([("parent", "<u2"), ("first_child", "<u2"), ("n_children", "u1"), ("kind_act", "u1"),
                       ("depth", "u1"), ("internal_idx", "u1"), ("v0", "<f4"), ("v1", "<f4")])
SUBGAME_DTYPE = np.dtype([("node_begin", "<i4"), ("n_nodes", "<i4"), ("n_internal", "<i4"), ("table_index", "<i4"),
                          ("scale", "<f4"), ("allowed_prob", "<f4"), ("board_mask", "<u8")])
SCALAR_DTYPE = np.dtype([("num_pos", "<f4"), ("den_pos", "<f4"), ("num_neg", "<f4"), ("den_neg", "<f4"),
                         ("mix_old", "<f4"), ("mix_new", "<f4"), ("mix_total", "<f4"), ("do_mix", "<i4")])
assert NODE_DTYPE.itemsize == 16 and SUBGAME_DTYPE.itemsize == 32 and SCALAR_DTYPE.itemsize == 32


def set_path_policy(policy: str) -> str:
    """Which kernel runs the iteration passes of one-call solves in this process: "auto" (default: the lean
    kernel except for batches so small that the general kernel is quicker, see `p2b_cfr_path_policy`) or "lean"
    (the lean kernel whenever it applies).  Returns the previous setting; results do not depend on it."""
    names = ("auto", "lean")
    if policy not in names:
        raise ValueError(f"unknown path policy {policy!r}")
    return names[int(_lib.lib().p2b_cfr_path_policy(names.index(policy)))]


def node_kind(records):
    """Kind of node records (`tree.KIND_*`): bits 0-1 of the `kind_act` byte."""
    return records["kind_act"] & 3


def node_to_act(records):
    """Player to act at node records: bit 7 of the `kind_act` byte."""
    return records["kind_act"] >> 7


def iteration_scalars(iterations: int, *, cfr_type: str = "discounted", alpha: float = 1.5, beta: float = 0.0,
                      gamma: float = 2.0, dcfr_delay: int = 0, alpha_final: float | None = None,
                      beta_final: float | None = None, gamma_final: float | None = None,
                      warm_start_iterations: int = 0) -> np.ndarray:
    """Per-iteration discount and mixing scalars for t = 0..iterations-1, evaluated in Python
    floats and rounded to fp32 exactly as the upstream loop does (cfr_evaluator.py:1346-1360,
    285-303, 1197-1205).  t is 0-based: 0**0.0 == 1 and 0**1.5 == 0.

    alpha / beta / gamma are the initial exponents; with a `*_final` value the exponent of
    iteration t is interpolated linearly over the iterations after the warm start, as
    `apply_schedules` does (cfr_evaluator.py:1294-1329):
    progress = clamp((t - warm_start_iterations) / max(1, iterations - warm_start_iterations), 0, 1).
    Rows below `warm_start_iterations` are never run by the upstream loop (it starts at the warm
    start, :1516); they are left at the neutral value 1 instead of evaluating t ** exponent there
    (0 ** negative raises in Python, which the production setting beta = -1 would hit at t = 0).
    The row AT `warm_start_iterations` also serves the warm start's own `update_policy(w)` call
    (:923), which upstream runs before any schedule is applied, i.e. with the initial gamma:
    `solver.SteppedSolver.solve` builds that extra pass from `warm_start_mix_scalars`."""
    if cfr_type not in ("standard", "discounted", "discounted_plus", "linear"):
        raise ValueError(f"unknown cfr_type {cfr_type!r}")
    ws = max(0, int(warm_start_iterations))
    out = np.zeros(iterations, dtype=SCALAR_DTYPE)
    discounted = cfr_type in ("discounted", "discounted_plus")
    span = max(1, iterations - ws)
    for t in range(iterations):
        if t < ws:  # never run: neutral scalars, average policy := current policy
            out[t]["num_pos"] = out[t]["den_pos"] = out[t]["num_neg"] = out[t]["den_neg"] = 1.0
            out[t]["mix_old"], out[t]["mix_new"], out[t]["mix_total"], out[t]["do_mix"] = 0.0, 1.0, 1.0, 0
            continue
        progress = min(1.0, max(0.0, max(0, t - ws) / float(span)))
        a_t = alpha if alpha_final is None else alpha + (alpha_final - alpha) * progress
        b_t = beta if beta_final is None else beta + (beta_final - beta) * progress
        g_t = gamma if gamma_final is None else gamma + (gamma_final - gamma) * progress
        if discounted:
            # integer base like upstream (`t**self.dcfr_alpha` with an int t): identical to float(t) ** x
            ta, tb = t ** a_t, t ** b_t
            out[t]["num_pos"], out[t]["den_pos"] = ta, ta + 1
            out[t]["num_neg"], out[t]["den_neg"] = tb, tb + 1
        else:
            out[t]["num_pos"] = out[t]["den_pos"] = out[t]["num_neg"] = out[t]["den_neg"] = 1.0
        old, new = _mixing_weights(cfr_type, t, g_t, dcfr_delay)
        out[t]["mix_old"], out[t]["mix_new"], out[t]["mix_total"] = old, new, old + new
        out[t]["do_mix"] = 0 if (t == 0 or (discounted and t <= dcfr_delay)) else 1
        if cfr_type == "linear":  # alternating updates: the actions of player t % 2 get no regret (:1348-1349)
            out[t]["do_mix"] |= ((t % 2) + 1) << 1
    return out


def _mixing_weights(cfr_type: str, t: int, gamma: float, dcfr_delay: int):
    """`_get_mixing_weights` (cfr_evaluator.py:285-303)."""
    if cfr_type == "standard":
        return t, 1
    if cfr_type == "linear":
        return t, 2
    if cfr_type == "discounted":
        return t ** gamma, (t + 1) ** gamma
    return (t - dcfr_delay, 2) if t > dcfr_delay else (0, 1)  # discounted_plus


def warm_start_mix_scalars(scalars: np.ndarray, *, cfr_type: str, gamma: float, dcfr_delay: int,
                           warm_start_iterations: int) -> np.ndarray:
    """The scalars of the extra pass a warm start adds in front of the iterations: the warm start
    ends with `update_policy(w)` (cfr_evaluator.py:923), whose average-policy mix uses t = w and
    the exponent gamma as it stands before any schedule was applied (the initial value).  The
    regret-discount fields of that pass are not used (the warm start seeds the regrets itself)."""
    w = int(warm_start_iterations)
    row = scalars[w:w + 1].copy()
    old, new = _mixing_weights(cfr_type, w, gamma, dcfr_delay)
    row["mix_old"], row["mix_new"], row["mix_total"] = old, new, old + new
    discounted = cfr_type in ("discounted", "discounted_plus")
    row["do_mix"] = (0 if (w == 0 or (discounted and w <= dcfr_delay)) else 1) | (int(row["do_mix"][0]) & 6)
    return row


@dataclass
class DeviceTreeLayout:
    """Subgame-major node order and the packed records the kernel reads."""

    subgames: np.ndarray  # [B] SUBGAME_DTYPE
    nodes: np.ndarray  # [rows] NODE_DTYPE
    to_level_major: np.ndarray  # [rows] level-major (upstream) index of each row
    from_level_major: np.ndarray  # [rows] row of each level-major node
    max_internal: int
    max_children: int
    tree_depth: int  # depth of the deepest tree of the batch
    # leaves valued by a model (start of the next street, depth limit), in slot order
    leaf_begin: np.ndarray = None  # [B] int32 first slot of each subgame
    model_rows: np.ndarray = None  # [slots] row of each model leaf
    model_nodes: np.ndarray = None  # [slots] level-major (upstream) node index of each model leaf

    @property
    def rows(self) -> int:
        return self.nodes.shape[0]

    @property
    def num_model_leaves(self) -> int:
        return 0 if self.model_rows is None else int(self.model_rows.shape[0])


def device_layout(trees: ptree.PublicTrees, boards: np.ndarray) -> DeviceTreeLayout:
    M, B = trees.total_nodes, trees.num_roots
    order = np.lexsort((np.arange(M), trees.root_of))  # by subgame, then upstream order (breadth-first)
    pos = np.empty(M, dtype=np.int64)
    pos[order] = np.arange(M)
    n_nodes = np.bincount(trees.root_of, minlength=B)
    node_begin = np.concatenate([[0], np.cumsum(n_nodes)])[:-1]
    if n_nodes.max() > MAX_NODES:
        raise ValueError(f"a subgame has {n_nodes.max()} nodes; the kernel supports up to {MAX_NODES}")
    if trees.child_count.max() > MAX_CHILDREN:
        raise ValueError(f"at most {MAX_CHILDREN} actions per node are supported")
    local = pos - node_begin[trees.root_of]
    st = trees.state
    internal = trees.child_count > 0
    fold = (trees.action_from_parent == 0) & st.done
    showdown = (st.street == 4) & ~internal
    kind = np.full(M, ptree.KIND_MODEL, dtype=np.uint8)
    kind[showdown] = ptree.KIND_SHOWDOWN
    kind[fold] = ptree.KIND_FOLD
    kind[internal] = ptree.KIND_INTERNAL
    rec = np.zeros(M, dtype=NODE_DTYPE)
    parent_local = np.where(trees.parent_index >= 0, local[np.maximum(trees.parent_index, 0)], 0)
    first_child = np.where(internal, local[np.minimum(trees.child_offsets, M - 1)], 0)
    rec["parent"], rec["first_child"] = parent_local, first_child
    rec["n_children"] = trees.child_count
    rec["kind_act"] = kind | (st.to_act.astype(np.uint8) << 7)
    rec["depth"] = trees.depth_of
    rec["v0"] = np.where(fold, trees.fold_value, trees.showdown_potential[:, 0].astype(np.float32))
    rec["v1"] = trees.showdown_potential[:, 1].astype(np.float32)
    rec = rec[order]
    # rank among the internal nodes of the same subgame
    int_sorted = internal[order].astype(np.int64)
    csum = np.cumsum(int_sorted) - int_sorted
    root_sorted = trees.root_of[order]
    rec["internal_idx"] = csum - csum[node_begin[root_sorted]]
    n_internal = np.bincount(trees.root_of, weights=internal, minlength=B).astype(np.int64)
    # model leaves: rank among the model leaves of the subgame, slots in row order
    is_model = node_kind(rec) == ptree.KIND_MODEL
    mdl = is_model.astype(np.int64)
    msum = np.cumsum(mdl) - mdl
    rec["internal_idx"] = np.where(is_model, msum - msum[node_begin[root_sorted]], rec["internal_idx"])
    n_model = np.bincount(root_sorted, weights=mdl, minlength=B).astype(np.int64)
    leaf_begin = (np.cumsum(n_model) - n_model).astype(np.int32)
    model_rows = np.nonzero(is_model)[0]

    boards = np.asarray(boards, dtype=np.int64)
    sub = np.zeros(B, dtype=SUBGAME_DTYPE)
    sub["node_begin"], sub["n_nodes"], sub["n_internal"] = node_begin, n_nodes, n_internal
    has_sd = np.bincount(trees.root_of, weights=showdown, minlength=B) > 0
    sub["table_index"] = np.where(has_sd, np.arange(B), -1)
    sub["scale"] = st.scale[:B]
    mask = np.zeros(B, dtype=np.uint64)
    n_blocked_cards = np.zeros(B, dtype=np.int64)
    for j in range(boards.shape[1]):
        valid = boards[:, j] >= 0
        mask[valid] |= np.uint64(1) << boards[valid, j].astype(np.uint64)
        n_blocked_cards += valid
    sub["board_mask"] = mask
    n_allowed = (52 - n_blocked_cards) * (51 - n_blocked_cards) // 2
    sub["allowed_prob"] = (np.float32(1.0) / np.maximum(n_allowed, 1).astype(np.float32)).astype(np.float32)
    return DeviceTreeLayout(subgames=sub, nodes=rec, to_level_major=order, from_level_major=pos,
                            max_internal=int(n_internal.max()), max_children=int(trees.child_count.max()),
                            tree_depth=trees.tree_depth, leaf_begin=leaf_begin, model_rows=model_rows,
                            model_nodes=order[model_rows])


def layout_tensor(layout, name: str, device, dtype=None) -> torch.Tensor:
    """Field `name` of a tree layout as a tensor on `device`: the device copy a layout built on
    the GPU already holds (`device_tree.DeviceBuiltLayout`), else an upload of the numpy array."""
    t = getattr(layout, name + "_dev", None)
    if t is None:
        t = torch.from_numpy(np.ascontiguousarray(getattr(layout, name)))
    t = t.to(device)
    return t if dtype is None else t.to(dtype)


def scalars_are_linear(scalars: np.ndarray) -> bool:
    """True if the table was made for linear CFR (some iteration skips a player's regrets)."""
    return bool((scalars["do_mix"] & 6).any())


def solve_flags(cfr_plus: bool, enforce_zero_sum: bool, cfr_avg: bool = False, iter_values: bool = False,
                linear: bool = False) -> int:
    """The `flags` argument of the solve entry points: bit 0 = CFR+ clamp, bit 1 = zero-sum value outputs,
    bit 2 = leaf values and regret weights at the beliefs under the average policy (`cfr_avg` upstream),
    bit 3 (stepped solves) = keep the node values and average beliefs of every pass, bit 4 = linear CFR (the
    scalars carry the skipped player; every pass in the general kernel)."""
    return (int(bool(cfr_plus)) | (int(bool(enforce_zero_sum)) << 1) | (int(bool(cfr_avg)) << 2)
            | (int(bool(iter_values)) << 3) | (int(bool(linear)) << 4))


def pad_rows(x: torch.Tensor) -> torch.Tensor:
    """[..., 1326] -> [..., 1344] zero padded (rows of the kernel are 16-byte aligned)."""
    out = x.new_zeros(*x.shape[:-1], HPAD)
    out[..., :NUM_HANDS] = x
    return out


@dataclass
class SolveResult:
    """Arrays in the kernel's subgame-major row order, padded to 1344 columns.  Use
    `level_major(x)` to obtain the upstream node order with 1326 columns."""

    layout: DeviceTreeLayout
    policy_avg: torch.Tensor  # [rows,1344]
    regrets: torch.Tensor  # [rows,1344]
    weight_sums: torch.Tensor | None
    policy: torch.Tensor | None
    root_values: torch.Tensor  # [B,2,1344]
    values_avg: torch.Tensor | None  # [rows,2,1344]
    beliefs_avg: torch.Tensor | None
    exploitability: torch.Tensor | None = None  # [B] local exploitability of the average policy
    br_values: torch.Tensor | None = None  # [B,2] best-response values at the roots
    policy_sample: torch.Tensor | None = None  # [rows,1344] policy of each subgame's sampling iteration
    beliefs_last: torch.Tensor | None = None  # [rows,2,1344] beliefs of the last iteration (internal nodes)

    def to_host(self, pinned: dict | None = None) -> dict:
        """Copies the training targets (root values, average policy) to pinned host memory
        and waits for the copy."""
        pinned = {} if pinned is None else pinned
        for name, src in (("root_values", self.root_values), ("policy_avg", self.policy_avg)):
            if name not in pinned or pinned[name].shape != src.shape:
                pinned[name] = torch.empty(src.shape, dtype=src.dtype, pin_memory=True)
            pinned[name].copy_(src, non_blocking=True)
        torch.cuda.current_stream(self.root_values.device).synchronize()
        return pinned

    def to_host_async(self, pinned: dict, copy_stream: "torch.cuda.Stream"):
        """Starts the copy of the training targets to pinned host memory on `copy_stream`, after the
        work already queued on the current stream; returns (pinned, event).  The targets are on the
        host once the event has completed; this object must stay alive until then.  Lets the copy of
        one batch run while the next batch is being solved."""
        dev = self.root_values.device
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(dev))
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(ready)
            for name, src in (("root_values", self.root_values), ("policy_avg", self.policy_avg)):
                if name not in pinned or pinned[name].shape != src.shape:
                    pinned[name] = torch.empty(src.shape, dtype=src.dtype, pin_memory=True)
                pinned[name].copy_(src, non_blocking=True)
            done = torch.cuda.Event()
            done.record(copy_stream)
        return pinned, done

    def level_major(self, x: torch.Tensor) -> torch.Tensor:
        return x.index_select(0, layout_tensor(self.layout, "from_level_major", x.device))[..., :NUM_HANDS]


class SubgameSolver:
    """Holds the device buffers of one batch shape and runs the fused kernel on them."""

    def __init__(self, layout: DeviceTreeLayout, boards: torch.Tensor, device: torch.device, *,
                 track_weight_sums: bool = True, keep_policy: bool = False, keep_node_values: bool = False,
                 exploitability: bool = False, num_blocks: int = 0, sampling: bool = False,
                 lean_iterations: bool = True):
        """lean_iterations=False gives the kernel only its minimal scratch area, which keeps every
        pass of a solve in the general kernel (one launch); results are the same bit for bit."""
        keep_node_values = keep_node_values or exploitability  # best responses read the node values
        if device.type != "cuda":
            raise ValueError("SubgameSolver requires a CUDA device.")
        self.layout, self.device = layout, device
        built_on_device = getattr(layout, "subgames_dev", None) is not None
        rows = layout.rows
        B = int(layout.subgames_dev.shape[0]) if built_on_device else layout.subgames.shape[0]
        self.B = B
        with torch.cuda.device(device):
            blocks = num_blocks if num_blocks > 0 else int(_lib.lib().p2b_cfr_default_blocks())
        self.num_blocks = min(blocks, B)
        f32 = dict(device=device, dtype=torch.float32)
        if built_on_device:
            self.subgames, self.nodes = layout.subgames_dev.to(device), layout.nodes_dev.to(device)
            has_showdown = layout.has_showdown
        else:
            self.subgames = torch.from_numpy(layout.subgames.view(np.uint8).reshape(B, 32)).to(device)
            self.nodes = torch.from_numpy(layout.nodes.view(np.uint8).reshape(rows, 16)).to(device)
            has_showdown = bool((layout.subgames["table_index"] >= 0).any())
        self.tables = BoardTables(boards.to(device)) if has_showdown else None
        # zeroed once: the kernel rewrites every non-root row on each solve and never touches
        # the root rows (a root is reached by no action)
        self.regrets = torch.zeros(rows, HPAD, **f32)
        self.policy_avg = torch.zeros(rows, HPAD, **f32)
        self.weight_sums = torch.zeros(rows, HPAD, **f32) if track_weight_sums else None
        self.policy = torch.zeros(rows, HPAD, **f32) if keep_policy else None
        self.root_values = torch.empty(B, 2, HPAD, **f32)
        self.values_avg = torch.zeros(rows, 2, HPAD, **f32) if keep_node_values else None
        self.beliefs_avg = torch.zeros(rows, 2, HPAD, **f32) if keep_node_values else None
        self.exploitability = torch.zeros(B, **f32) if (exploitability and keep_node_values) else None
        self.br_values = torch.zeros(B, 2, **f32) if (exploitability and keep_node_values) else None
        # the larger area lets a solve without optional outputs run its iteration passes in the lean kernel
        if lean_iterations:
            n_scratch = int(_lib.lib().p2b_cfr_solve_scratch_floats(layout.max_internal, layout.max_children,
                                                                    self.num_blocks, B, rows))
        else:
            n_scratch = int(_lib.lib().p2b_cfr_scratch_floats(layout.max_internal, self.num_blocks))
        self.scratch = torch.empty(n_scratch, **f32)
        self.work_counter = torch.zeros(4, device=device, dtype=torch.int32)
        # the thread blocks take subgames from a queue: largest trees first, so that the blocks that finish
        # last hold small ones (a stable sort: equal sizes keep their input order)
        if built_on_device:
            n_nodes = self.subgames.view(torch.int32).reshape(B, 8)[:, 1]
        else:
            n_nodes = torch.from_numpy(np.ascontiguousarray(layout.subgames["n_nodes"])).to(device)
        self.queue_order = torch.argsort(n_nodes, descending=True, stable=True).to(torch.int32).contiguous()
        # leaf sampling: the policy of one scheduled iteration per subgame, beliefs of the last one
        self.policy_sample = torch.zeros(rows, HPAD, **f32) if sampling else None
        self.beliefs_last = torch.zeros(rows, 2, HPAD, **f32) if sampling else None
        self.sample_pass = torch.full((B,), -2, device=device, dtype=torch.int32) if sampling else None
        self.launches = 0

    def set_sampling_schedule(self, t_sample: torch.Tensor, warm_start_iterations: int = 0) -> None:
        """t_sample [B]: iteration at whose start each subgame's current policy is kept
        (`sampling.sampling_schedule`).  The policy at the start of iteration t is the policy of
        pass t-1; after a warm start of w iterations pass k >= 1 runs iteration w+k-1, so it is
        the policy of pass t-w."""
        if self.sample_pass is None:
            raise ValueError("the solver was built without sampling=True")
        shift = warm_start_iterations if warm_start_iterations > 0 else 1
        self.sample_pass.copy_((t_sample.to(torch.int64) - shift).to(torch.int32))
        self.policy_sample.zero_()

    def _result(self) -> "SolveResult":
        return SolveResult(self.layout, self.policy_avg, self.regrets, self.weight_sums, self.policy,
                           self.root_values, self.values_avg, self.beliefs_avg, self.exploitability, self.br_values,
                           self.policy_sample, self.beliefs_last)

    def status(self) -> int:
        """0, or 1 + the index of a subgame whose records exceed the kernel's limits, in which
        case the last solve did nothing.  Reads one word from the device (synchronises)."""
        return int(self.work_counter[1].item())

    def release(self) -> None:
        """Drops the device buffers (they return to the caching allocator)."""
        for name in ("regrets", "policy_avg", "weight_sums", "policy", "root_values", "values_avg", "beliefs_avg",
                     "exploitability", "br_values", "scratch", "tables", "policy_sample", "beliefs_last", "_graphed"):
            setattr(self, name, None)

    def solve(self, root_beliefs: torch.Tensor, scalars: np.ndarray, *, cfr_plus: bool = False,
              enforce_zero_sum: bool = False, cfr_avg: bool = False, check: bool = False,
              start_policy: torch.Tensor | None = None, warm_start_iterations: int = 0,
              warm_start_multiplier: float = 1.0, warm_start_scalars: np.ndarray | None = None) -> SolveResult:
        """root_beliefs: [B,2,1344] fp32 on the device (padded).  Enqueues the solve (one to three
        kernels, one more for a warm start).  start_policy [M,1326] in the upstream node order (the policy head's
        soft-max; None = uniform); with warm_start_iterations = w > 0 the regrets are seeded from it after the
        start pass (`warm_start` of type `model`, cfr_evaluator.py:887-926) and iterations w..T-1 follow, as in
        `SteppedSolver.solve` (same meaning of `scalars` and `warm_start_scalars`).  enforce_zero_sum: shift the value outputs to zero sum, as upstream does when
        `model.enforce_zero_sum` is set (cfr_evaluator.py:957-980, 1289-1292).  cfr_avg: showdown values
        and regret weights at the beliefs under the average policy (:1029, :1133; one launch, general
        kernel).  check: read the status word afterwards (synchronises) and raise if the record check
        refused the batch."""
        assert root_beliefs.shape == (self.B, 2, HPAD) and root_beliefs.dtype == torch.float32
        assert root_beliefs.is_contiguous() and root_beliefs.device == self.device
        ws = int(warm_start_iterations)
        if ws > 0:
            if start_policy is None:
                raise ValueError("a warm start needs a start policy")
            first = scalars[ws:ws + 1] if warm_start_scalars is None else warm_start_scalars
            scalars = np.concatenate([first, scalars[ws:]])
        start_rows = None
        if start_policy is not None:
            order = layout_tensor(self.layout, "to_level_major", start_policy.device)
            start_rows = pad_rows(start_policy.to(torch.float32)[order]).to(self.device).contiguous()
        self._start_rows = start_rows  # alive until the kernels have run
        iterations = int(scalars.shape[0])
        sc = torch.from_numpy(scalars.view(np.uint8).reshape(max(iterations, 0), 32).copy()).to(self.device)
        self._scalars = sc
        p = _lib.ptr
        with torch.cuda.device(self.device):
            _lib.call(
                "p2b_cfr_solve", p(self.subgames), p(self.nodes), self.B, self.layout.rows, self.layout.max_children,
                self.layout.max_internal, p(self.tables.blob) if self.tables is not None else None, p(root_beliefs),
                p(self.regrets), p(self.weight_sums), p(self.policy_avg), p(self.policy), p(self.root_values),
                p(self.values_avg), p(self.beliefs_avg), p(self.exploitability), p(self.br_values), p(self.scratch),
                self.scratch.numel(),
                p(sc) if iterations else None, iterations,
                solve_flags(cfr_plus, enforce_zero_sum, cfr_avg, linear=scalars_are_linear(scalars)),
                self.layout.tree_depth, p(self.work_counter),
                self.num_blocks, p(self.sample_pass), p(self.policy_sample), p(self.beliefs_last),
                p(self.queue_order), p(start_rows), float(ws) * float(warm_start_multiplier) if ws > 0 else 0.0,
                _lib.stream_ptr(self.device))
        self.launches += 1
        if check:
            self.raise_if_refused()
        return self._result()

    def raise_if_refused(self) -> None:
        st = self.status()
        if st != 0:
            raise RuntimeError(f"subgame {st - 1}: tree records exceed the solver's limits; nothing was solved")


class SteppedSolver(SubgameSolver):
    """Solves subgames whose non-terminal leaves are valued by a caller-side model
    (`set_leaf_values`, p2/search/cfr_evaluator.py:1025-1047): every pass is two launches
    (`p2b_cfr_step`) with the model call in between.

    `leaf_fn(beliefs)` receives the beliefs at the model leaves, [slots,2,1344] fp32 on the
    device (columns 1326.. are padding; slot order = `layout.model_rows`), and returns their
    values for both players in the same shape (or [slots,2,1326]), in chips / scale."""

    def __init__(self, layout: DeviceTreeLayout, boards: torch.Tensor, device: torch.device, **kw):
        super().__init__(layout, boards, device, **kw)
        f32 = dict(device=device, dtype=torch.float32)
        n_scratch = int(_lib.lib().p2b_cfr_scratch_floats(layout.max_internal, 1)) * self.B
        self.scratch = torch.empty(n_scratch, **f32)
        self.carry_sums = torch.zeros(2, layout.rows, 2, **f32)  # current-policy sums, average-policy sums
        self.carry_roots = torch.zeros(self.B, 4, HPAD, **f32)
        slots = max(layout.num_model_leaves, 1)
        self.leaf_begin = layout_tensor(layout, "leaf_begin", device, torch.int32)
        self.leaf_beliefs = torch.zeros(slots, 2, HPAD, **f32)
        self.leaf_values = torch.zeros(slots, 2, HPAD, **f32)

    start_policy_rows = None  # [rows,1344] policy of the start pass (None: uniform)
    _last_model_values = None
    _graphed = None  # (key, GraphedPass) of the last solve with graph=True

    def _de_average(self, vals, t, scalars, enforce_zero_sum, n_leaves):
        """The CFR-AVG branch of `_set_model_values_impl` (cfr_evaluator.py:997-1018): from t = 2 on the
        model's values are read as the average over the iterations, so this iteration's are
        ((old + new) * values - old * last) / new, shifted to zero sum by the leaf beliefs if asked."""
        raw = vals[..., :NUM_HANDS].to(torch.float32)
        last, self._last_model_values = self._last_model_values, raw.clone()
        if t <= 1 or last is None:
            return vals
        row = scalars[t]
        old, total = float(row["mix_old"]), float(row["mix_total"])
        new = torch.tensor(float(row["mix_new"]), device=raw.device, dtype=torch.float32)
        unmixed = (total * raw - old * last) / new  # a tensor divisor: an IEEE division, like the CPU's
        if enforce_zero_sum:
            from . import fused_cfr as F

            one, zero = (torch.tensor(v, device=raw.device, dtype=torch.float32) for v in (1.0, 0.0))
            out = torch.empty_like(unmixed)
            # unmixed * 1 - 0 * 0 is unmixed itself; the kernel adds the shift, its sums in the CPU's order
            F.mix_zero_sum(unmixed.contiguous(), torch.zeros_like(unmixed),
                           self.leaf_beliefs[:n_leaves, :, :NUM_HANDS].contiguous(), one, zero, out, mode=2)
            unmixed = out
        return unmixed

    def _step(self, root_beliefs, sc, iterations, flags, pass_begin, pass_end, phases, sample_pass=None) -> None:
        p = _lib.ptr
        if sample_pass is None:
            sample_pass = self.sample_pass
        with torch.cuda.device(self.device):
            _lib.call(
                "p2b_cfr_step", p(self.subgames), p(self.nodes), self.B, self.layout.rows, self.layout.max_children,
                self.layout.max_internal, p(self.tables.blob) if self.tables is not None else None, p(root_beliefs),
                p(self.regrets), p(self.weight_sums), p(self.policy_avg), p(self.policy), p(self.root_values),
                p(self.values_avg), p(self.beliefs_avg), p(self.exploitability), p(self.br_values), p(self.scratch),
                self.scratch.numel(), p(sc), iterations, int(flags), self.layout.tree_depth, p(self.work_counter),
                self.num_blocks, pass_begin, pass_end, phases, p(self.carry_sums), p(self.carry_roots),
                p(self.leaf_begin), int(self.leaf_beliefs.shape[0]), p(self.leaf_beliefs), p(self.leaf_values),
                p(sample_pass),
                p(self.policy_sample), p(self.beliefs_last), p(self.queue_order), p(self.start_policy_rows),
                _lib.stream_ptr(self.device))
        self.launches += 1

    def solve(self, root_beliefs: torch.Tensor, scalars: np.ndarray, leaf_fn=None, *, cfr_plus: bool = False,
              enforce_zero_sum: bool = False, start_policy: torch.Tensor | None = None, warm_start_iterations: int = 0,
              warm_start_multiplier: float = 1.0, warm_start_scalars: np.ndarray | None = None,
              cfr_avg: bool = False, running_values: bool = False, warm_start_type: str = "model",
              policy_delta=None, graph: bool = False, joint_sweeps: bool = False) -> SolveResult:
        """scalars: `iteration_scalars(T)` for all T iterations.  start_policy [M,1326] in the
        upstream node order (the policy head's softmax; None = uniform).  With
        warm_start_iterations = w > 0 (needs a start policy) the regrets are seeded from the start
        policy after the start pass (`warm_start` of type `model`, cfr_evaluator.py:887-926) and
        the iterations w..T-1 follow; `warm_start_scalars` (one row, `warm_start_mix_scalars`) gives
        the mixing weights of the warm start's own policy update when the exponents follow a
        schedule (default: the row of iteration w).  cfr_avg: `cfr_avg` upstream -- leaf_fn sees the
        beliefs under the average policy, and from the second iteration on its values are taken as a
        running average over the iterations and de-averaged (cfr_evaluator.py:997-1018).
        running_values: `value_targets_from_final_policy = False` upstream -- the value outputs are the
        running mix of the per-iteration node values, shifted to zero sum every iteration if asked
        (`update_average_values`, :1260-1274), instead of the values of the final average policy; the
        solver must have been built with keep_node_values=True (or exploitability=True).
        warm_start_type: "model" (above) or "model_br" (:927-955; needs keep_node_values too): the regrets
        are seeded with w x multiplier x the regrets of not playing a best response against the start
        policy.
        policy_delta: a `stats.PolicyDelta` of this batch -- the change of the current policy at the five
        iterations of `stats.delta_checkpoints` is left in `self.policy_deltas` (percentile -> 0-dim device
        tensor), from the regrets on either side of those iterations' updates (`_record_stats`,
        cfr_evaluator.py:1573-1605).
        graph: replay the iteration passes 1..T-2 from one CUDA graph (`GraphedPass`) instead of
        launching their kernels and the leaf model's one by one; same kernels, same results.  Ignored
        where the host works between the passes (cfr_avg, running_values, policy_delta).  The leaf model must
        be capturable: device work only, the same shapes every pass, no host synchronisation.
        joint_sweeps: with model leaves, launch the bottom-up sweep of a pass together with the top-down sweep
        of the next one (`phases` 16 of `p2b_cfr_step`) wherever the host has nothing to do between them, so
        that a pass is one solver launch instead of two; same results.  Off by default: measured on 192
        flop subgames of 273 nodes it changes nothing (2.50 against 2.47 ms per pass), the time of a pass is
        the blocks' walk over the subgames, not the launches."""
        assert root_beliefs.shape == (self.B, 2, HPAD) and root_beliefs.dtype == torch.float32
        assert root_beliefs.is_contiguous() and root_beliefs.device == self.device
        ws = int(warm_start_iterations)
        flags = solve_flags(cfr_plus, enforce_zero_sum, cfr_avg, running_values, linear=scalars_are_linear(scalars))
        if running_values and self.values_avg is None:
            raise ValueError("running_values needs a solver built with keep_node_values=True")
        if warm_start_type not in ("model", "model_br"):
            raise ValueError(f"unknown warm_start_type {warm_start_type!r}")
        warm_br = ws > 0 and warm_start_type == "model_br"
        if warm_br and self.values_avg is None:
            raise ValueError("a warm start of type model_br needs a solver built with keep_node_values=True")
        all_scalars = scalars
        if ws > 0:
            if start_policy is None:
                raise ValueError("a warm start needs a start policy")
            # pass 0 is warm_start's own update_policy(w): it mixes with t = w, like iteration w after it
            first = scalars[ws:ws + 1] if warm_start_scalars is None else warm_start_scalars
            scalars = np.concatenate([first, scalars[ws:]])
        self.start_policy_rows = None
        if start_policy is not None:
            order = layout_tensor(self.layout, "to_level_major", start_policy.device)
            self.start_policy_rows = pad_rows(start_policy.to(torch.float32)[order]).to(self.device).contiguous()
        iterations = int(scalars.shape[0])
        sc = torch.from_numpy(scalars.view(np.uint8).reshape(iterations, 32).copy()).to(self.device)
        self._scalars = sc
        n_leaves = self.layout.num_model_leaves
        if n_leaves and leaf_fn is None:
            raise ValueError("the trees have model-valued leaves: a leaf_fn is required")
        self._last_model_values = None
        self._running = None
        self.policy_deltas = {}
        graphed = None
        if graph and not (cfr_avg or running_values or policy_delta is not None) and iterations >= 4:
            # a graph is tied to the addresses and settings it was captured with: kept across solves that share them
            key = (root_beliefs.data_ptr(), iterations, flags, id(leaf_fn))
            if self._graphed is None or self._graphed[0] != key:
                self._graphed = (key, GraphedPass(self, root_beliefs, sc, iterations, flags, leaf_fn))
            graphed = self._graphed[1]
            graphed.scalars = sc
        delta_at = {}
        if policy_delta is not None:
            from . import stats as pstats

            # the regret update of upstream iteration t happens in the bottom-up sweep of the pass before
            # the one that plays the updated policy: the start pass for iteration 0, pass t - w after a
            # warm start (whose pass 0 is the warm start's own policy update)
            for t, q in pstats.delta_checkpoints(ws, all_scalars.shape[0]).items():
                delta_at[t - ws + (0 if ws > 0 else -1)] = q
        # the bottom-up sweep of a pass waits for the top-down sweep of the next one where they can share a launch
        fuse = (joint_sweeps and n_leaves > 0 and graphed is None
                and not (cfr_avg or running_values or policy_delta is not None))
        pending_up = None
        for pas in range(-1, iterations + 1):
            if pas == 0 and warm_br:
                # best responses against the start policy, from the node values the start pass has stored
                self._step(root_beliefs, sc, iterations, flags, -1, -1, 8)
                weight = float(ws) * float(warm_start_multiplier)
                self.regrets.mul_(weight)
                if self.weight_sums is not None:
                    self.weight_sums.fill_(weight)
            elif pas == 0 and ws > 0:
                with torch.cuda.device(self.device):
                    _lib.call("p2b_cfr_warm_seed", _lib.ptr(self.nodes), self.layout.rows, _lib.ptr(self.start_policy_rows),
                              float(ws) * float(warm_start_multiplier), _lib.ptr(self.regrets), _lib.ptr(self.weight_sums),
                              _lib.stream_ptr(self.device))
                self.launches += 1
            if running_values and pas == iterations:
                self._finish_running_values(root_beliefs, sc, iterations, flags, leaf_fn, n_leaves)
                break
            if pas == -1 and warm_br:
                flags_pass = flags | 8  # the start pass keeps its node values for the best responses
            else:
                flags_pass = flags
            if graphed is not None and 1 <= pas <= iterations - 2:
                if graphed.captured_t is None:
                    graphed.capture(pas)  # passes -1 and 0 have run: every lazy set-up is done
                graphed.replay(pas)
                continue
            before = None
            if pas in delta_at:  # the policy this pass plays; its bottom-up sweep updates the regrets
                before = policy_delta.start_policy(start_policy) if pas < 0 else policy_delta.policy_of(self.regrets)
            if n_leaves == 0:
                self._step(root_beliefs, sc, iterations, flags_pass, pas, pas, 3)
                if running_values:
                    self._mix_running_values(pas, ws, all_scalars, enforce_zero_sum)
                if before is not None:
                    self.policy_deltas[delta_at[pas]] = policy_delta(before, policy_delta.policy_of(self.regrets))
                continue
            if pending_up is not None:
                self._step(root_beliefs, sc, iterations, flags_pass, pending_up, pas, 16)
                pending_up = None
            else:
                self._step(root_beliefs, sc, iterations, flags_pass, pas, pas, 1)
            vals = leaf_fn(self.leaf_beliefs[:n_leaves])
            if cfr_avg:
                # iteration the pass belongs to, as `set_leaf_values(t)` sees it: the start pass, the pass
                # that follows a warm start and the final pass pass t = 0 (:1511, :1288)
                t = 0 if (pas < 0 or pas == iterations) else (pas if ws == 0 else (0 if pas == 0 else ws + pas - 1))
                vals = self._de_average(vals, t, all_scalars, enforce_zero_sum, n_leaves)
            if vals.shape[-1] == NUM_HANDS:
                self.leaf_values[:n_leaves, :, :NUM_HANDS].copy_(vals)
            else:
                self.leaf_values[:n_leaves].copy_(vals)
            if self.beliefs_last is not None and pas == iterations - 1:
                # beliefs of the last iteration at the model leaves (the states sampling continues from)
                self.beliefs_last[layout_tensor(self.layout, "model_rows", self.device)] = self.leaf_beliefs[:n_leaves]
            if fuse and pas < iterations and not (pas == -1 and ws > 0):  # (a warm start seeds the regrets before pass 0)
                pending_up = pas
                continue
            self._step(root_beliefs, sc, iterations, flags_pass, pas, pas, 2)
            if running_values:
                self._mix_running_values(pas, ws, all_scalars, enforce_zero_sum)
            if before is not None:
                self.policy_deltas[delta_at[pas]] = policy_delta(before, policy_delta.policy_of(self.regrets))
        return self._result()

    # ---- running average of the node values (`value_targets_from_final_policy = False`) ----
    _running = None  # [rows,2,1344] the running average
    _terminal = None  # [rows] uint8: 1 at the leaves that end the hand (exempt from the zero-sum shift)

    def _mix_running_values(self, pas, ws, scalars, enforce_zero_sum) -> None:
        """After the bottom-up sweep of pass `pas` (whose node values are in self.values_avg, the average
        beliefs in self.beliefs_avg): the start pass, or the pass that follows a warm start, sets the
        average to the values (cfr_evaluator.py:1513); an iteration pass mixes them in with the weights
        of its iteration and shifts the result to zero sum (:1260-1274)."""
        from . import fused_cfr as F

        first = 0 if ws > 0 else -1
        if pas < first:
            return
        if pas == first:
            self._running = self.values_avg.clone()
            return
        t = pas if ws == 0 else ws + pas - 1
        row = scalars[t]
        dev = self.device
        old, new, total = (torch.tensor(float(row[k]), device=dev, dtype=torch.float32)
                           for k in ("mix_old", "mix_new", "mix_total"))
        if self._terminal is None:
            kind = self.nodes.view(torch.uint8).reshape(-1, 16)[:, 5] & 3  # the kind_act byte of every record
            self._terminal = ((kind == 1) | (kind == 2)).to(torch.uint8).contiguous()
        out = torch.empty_like(self._running)
        F.mix_zero_sum_rows(self._running, self.values_avg, self.beliefs_avg, self._terminal, old, new, total, out,
                            divide=True, mode=2 if enforce_zero_sum else 0)
        self._running = out

    def _finish_running_values(self, root_beliefs, sc, iterations, flags, leaf_fn, n_leaves) -> None:
        """No final evaluation of the average policy in this mode: the final pass still runs, because the
        best responses start from its reach rows and normalisation sums, but its values go to a scratch
        copy; the outputs are the running averages."""
        running = self._running
        keep = self.values_avg
        flags_final = flags & ~8
        expl = self.exploitability
        self.exploitability = None  # the best responses come later, from the running averages
        if n_leaves == 0:
            self._step(root_beliefs, sc, iterations, flags_final, iterations, iterations, 3)
        else:
            self._step(root_beliefs, sc, iterations, flags_final, iterations, iterations, 1)
            vals = leaf_fn(self.leaf_beliefs[:n_leaves])
            if vals.shape[-1] == NUM_HANDS:
                self.leaf_values[:n_leaves, :, :NUM_HANDS].copy_(vals)
            else:
                self.leaf_values[:n_leaves].copy_(vals)
            self._step(root_beliefs, sc, iterations, flags_final, iterations, iterations, 2)
        self.exploitability = expl
        self.values_avg = running
        roots = layout_tensor(self.layout, "from_level_major", self.device)[: self.B]
        self.root_values.copy_(running.index_select(0, roots))
        if expl is not None:
            self._step(root_beliefs, sc, iterations, flags_final, iterations, iterations, 4)
        del keep


class GraphedPass:
    """One iteration pass of a `SteppedSolver` (top-down sweep, the leaf model, bottom-up sweep) captured in
    a CUDA graph and replayed for the other iterations: the counterpart of upstream's
    `GraphedCFRIteration` (p2/search/fused_cfr_triton.py:2359-2457), which captures `cfr_iteration` and
    refreshes its device scalars (`TScalars`) outside the captured region before every replay.

    Here the kernels take the pass number by value, so the graph is captured as pass 0 of a table window:
    before a replay for pass t the rows t and t+1 of the discount / mixing table are copied into a
    two-row device buffer the captured launches read as rows 0 and 1, and the passes at which subgames
    keep their sampling policy are shifted by t the same way.  A pass in the window must be an ordinary
    one: 1 <= t <= iterations - 2 (the start pass, pass 0 after it, the last iteration and the final
    pass take other branches in the kernels and run as plain launches).  Tree records, state arrays and
    the root beliefs tensor are baked in at capture time, as upstream."""

    def __init__(self, sv: "SteppedSolver", root_beliefs: torch.Tensor, scalars_dev: torch.Tensor, iterations: int,
                 flags: int, leaf_fn=None):
        if sv.device.type != "cuda":
            raise ValueError("GraphedPass requires a CUDA solver.")
        if iterations < 4:
            raise ValueError("nothing to replay: fewer than four iterations")
        self.sv, self.root_beliefs, self.scalars, self.iterations = sv, root_beliefs, scalars_dev, int(iterations)
        self.flags, self.leaf_fn = int(flags), leaf_fn
        self.window = torch.zeros(2, 32, dtype=torch.uint8, device=sv.device)
        self.sample_window = None if sv.sample_pass is None else torch.full_like(sv.sample_pass, -2)
        self._graph = None
        self._captured_t = None
        self._launches = 0

    def _refresh(self, t: int) -> None:
        self.window.copy_(self.scalars[t:t + 2])
        if self.sample_window is not None:
            torch.sub(self.sv.sample_pass, int(t), out=self.sample_window)

    def _pass(self) -> None:
        sv, n_leaves = self.sv, self.sv.layout.num_model_leaves
        args = (self.root_beliefs, self.window, self.iterations, self.flags, 0, 0)
        if n_leaves == 0:
            sv._step(*args, 3, sample_pass=self.sample_window)
            return
        sv._step(*args, 1, sample_pass=self.sample_window)
        vals = self.leaf_fn(sv.leaf_beliefs[:n_leaves])
        if vals.shape[-1] == NUM_HANDS:
            sv.leaf_values[:n_leaves, :, :NUM_HANDS].copy_(vals)
        else:
            sv.leaf_values[:n_leaves].copy_(vals)
        sv._step(*args, 2, sample_pass=self.sample_window)

    def capture(self, t_capture: int) -> None:
        """Records the graph; nothing runs and the solver state does not move.  The solver must have run
        at least one pass with the same leaf model before (lazy set-up happens there, not under capture)."""
        if not 1 <= t_capture <= self.iterations - 2:
            raise ValueError("only the passes 1..iterations-2 can be captured")
        if self.sv.layout.num_model_leaves and self.leaf_fn is None:
            raise ValueError("the trees have model-valued leaves: a leaf_fn is required")
        self._refresh(t_capture)
        before = self.sv.launches
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.device(self.sv.device), torch.cuda.graph(graph):
            self._pass()
        self._launches, self.sv.launches = self.sv.launches - before, before
        self._graph, self._captured_t = graph, int(t_capture)

    def replay(self, t: int) -> None:
        if self._graph is None:
            raise RuntimeError("capture() must be called before replay().")
        if not 1 <= t <= self.iterations - 2:
            raise ValueError("only the passes 1..iterations-2 can be replayed")
        self._refresh(t)
        self._graph.replay()
        self.sv.launches += self._launches

    @property
    def captured_t(self):
        return self._captured_t


def solve_noalloc(sv: SubgameSolver, root_beliefs: torch.Tensor, scalars_dev: torch.Tensor, *,
                  cfr_plus: bool = False, enforce_zero_sum: bool = False) -> SolveResult:
    """Runs the same solve as `SubgameSolver.solve` through `p2b_cfr_solve_noalloc`, the entry
    point for hosts that cannot allocate GPU memory (a worker confined to a fixed memory
    slice, a latency-critical loop, a process whose framework pool owns all free memory).
    The library's built-in 32 MiB work area replaces `sv.scratch` and `sv.work_counter`;
    nothing is allocated here either: `scalars_dev` is the caller's device copy of the
    per-iteration scalars ([T,32] uint8) and outputs go to the buffers `sv` already owns.
    Calls share that work area, so do not overlap two of them on one GPU."""
    assert root_beliefs.shape == (sv.B, 2, HPAD) and root_beliefs.is_contiguous()
    p = _lib.ptr
    with torch.cuda.device(sv.device):
        _lib.call(
            "p2b_cfr_solve_noalloc", p(sv.subgames), p(sv.nodes), sv.B, sv.layout.rows, sv.layout.max_children,
            sv.layout.max_internal, p(sv.tables.blob) if sv.tables is not None else None, p(root_beliefs),
            p(sv.regrets), p(sv.weight_sums), p(sv.policy_avg), p(sv.policy), p(sv.root_values), p(sv.values_avg),
            p(sv.beliefs_avg), p(sv.exploitability), p(sv.br_values), p(scalars_dev), int(scalars_dev.shape[0]),
            solve_flags(cfr_plus, enforce_zero_sum), sv.layout.tree_depth,
            _lib.stream_ptr(sv.device))
    return SolveResult(sv.layout, sv.policy_avg, sv.regrets, sv.weight_sums, sv.policy, sv.root_values,
                       sv.values_avg, sv.beliefs_avg, sv.exploitability, sv.br_values)


def noalloc_status(device) -> int:
    """Verdict of the record check of the last `solve_noalloc` on `device`: 0, or 1 + the index of a
    subgame whose records were refused (that call then solved nothing).  Waits for the current
    stream; allocates nothing on the device."""
    import ctypes

    device = torch.device(device)
    out = ctypes.c_int32(-1)
    with torch.cuda.device(device):
        _lib.call("p2b_cfr_noalloc_status", ctypes.byref(out), _lib.stream_ptr(device))
    return int(out.value)


def solve_subgames(boards, ranges, pot, stacks, *, iterations: int, bet_bins=(0.5, 1.0), max_depth: int = 8,
                   max_raises=None, bb: int = 2, cfr_type: str = "discounted", alpha: float = 1.5, beta: float = 0.0,
                   gamma: float = 2.0, dcfr_delay: int = 0, cfr_plus: bool = False, device=None,
                   keep_policy: bool = False, keep_node_values: bool = False, track_weight_sums: bool = True,
                   exploitability: bool = False, device_tree: bool = False, enforce_zero_sum: bool = False,
                   alpha_final=None, beta_final=None, gamma_final=None, cfr_avg: bool = False,
                   lean_iterations: bool = True):
    """Solves a batch of river subgames: boards [B,5] card ids, ranges [B,2,1326] fp32,
    pot [B] and stacks [B] or [B,2] in chips.  Returns (SolveResult, PublicTrees); with
    `device_tree` the trees are expanded on the GPU (`device_tree.build_device_layout`), no host
    tree exists and the second value is None (the layout is `result.layout`)."""
    device = torch.device(device if device is not None else "cuda:0")
    boards_np = np.asarray(boards.cpu() if torch.is_tensor(boards) else boards, dtype=np.int64)
    pot_np = np.asarray(pot.cpu() if torch.is_tensor(pot) else pot, dtype=np.int64)
    stacks_np = np.asarray(stacks.cpu() if torch.is_tensor(stacks) else stacks, dtype=np.int64)
    roots = ptree.root_states(pot_np, stacks_np, min_raise=bb)
    if device_tree:
        from .device_tree import build_device_layout
        trees = None
        layout = build_device_layout(roots, boards_np, list(bet_bins), max_depth, bb=bb, max_raises=max_raises,
                                     device=device)
    else:
        trees = ptree.build_trees(roots, list(bet_bins), max_depth, bb=bb, max_raises=max_raises)
        layout = device_layout(trees, boards_np)
    solver = SubgameSolver(layout, torch.from_numpy(boards_np), device, track_weight_sums=track_weight_sums,
                           keep_policy=keep_policy, keep_node_values=keep_node_values, exploitability=exploitability,
                           lean_iterations=lean_iterations)
    rb = pad_rows(torch.as_tensor(ranges, dtype=torch.float32).to(device)).contiguous()
    scal = iteration_scalars(iterations, cfr_type=cfr_type, alpha=alpha, beta=beta, gamma=gamma, dcfr_delay=dcfr_delay,
                             alpha_final=alpha_final, beta_final=beta_final, gamma_final=gamma_final)
    return solver.solve(rb, scal, cfr_plus=cfr_plus, enforce_zero_sum=enforce_zero_sum, cfr_avg=cfr_avg), trees


def solve_subgames_with_model(boards, ranges, pot, stacks, model, *, street: int, iterations: int,
                              bet_bins=(0.5, 1.0), max_depth: int = 8, max_raises=None, bb: int = 2,
                              cfr_type: str = "discounted", alpha: float = 1.5, beta: float = 0.0, gamma: float = 2.0,
                              dcfr_delay: int = 0, cfr_plus: bool = False, device=None, chance_average: bool = True,
                              chunk: int = 2048, exploitability: bool = False, keep_node_values: bool = False,
                              device_tree: bool = False, enforce_zero_sum: bool = False, cfr_avg: bool = False,
                              graph: bool = False):
    """Solves a batch of flop (street=1, 3 board cards) or turn (street=2, 4 cards) subgames
    whose leaves at the start of the next street are valued by `model(beliefs, boards,
    context)`, averaged over the next public card when `chance_average` (the
    `single_card_chance_values` semantics).  Returns (SolveResult, PublicTrees, SteppedSolver);
    with `device_tree` the trees and the leaf context are built on the GPU and the second value
    is None."""
    from . import leaf_eval

    device = torch.device(device if device is not None else "cuda:0")
    boards_np = np.asarray(boards.cpu() if torch.is_tensor(boards) else boards, dtype=np.int64)
    if boards_np.shape[1] < 5:
        boards_np = np.concatenate([boards_np, np.full((boards_np.shape[0], 5 - boards_np.shape[1]), -1)], axis=1)
    pot_np = np.asarray(pot.cpu() if torch.is_tensor(pot) else pot, dtype=np.int64)
    stacks_np = np.asarray(stacks.cpu() if torch.is_tensor(stacks) else stacks, dtype=np.int64)
    roots = ptree.root_states(pot_np, stacks_np, min_raise=bb, street=street)
    if device_tree:
        from .device_tree import build_device_layout
        trees = None
        layout = build_device_layout(roots, boards_np, list(bet_bins), max_depth, bb=bb, max_raises=max_raises,
                                     device=device, node_state=True)
    else:
        trees = ptree.build_trees(roots, list(bet_bins), max_depth, bb=bb, max_raises=max_raises)
        layout = device_layout(trees, boards_np)
    sv = SteppedSolver(layout, torch.from_numpy(boards_np), device, exploitability=exploitability,
                       keep_node_values=keep_node_values)
    if device_tree:
        leaf_boards = torch.from_numpy(boards_np).to(device)[layout.root_of_row_dev[layout.model_rows_dev]]
        ctx = layout.leaf_context()
    else:
        leaf_boards = torch.from_numpy(boards_np[trees.root_of[layout.model_nodes]])
        ctx = leaf_eval.leaf_context(trees, layout.model_nodes)
    if chance_average:
        evaluator = leaf_eval.ChanceLeafEvaluator(model, leaf_boards, ctx, device, chunk=chunk)
    else:
        evaluator = leaf_eval.DirectLeafEvaluator(model, leaf_boards, ctx, device)
    rb = pad_rows(torch.as_tensor(ranges, dtype=torch.float32).to(device)).contiguous()
    scal = iteration_scalars(iterations, cfr_type=cfr_type, alpha=alpha, beta=beta, gamma=gamma, dcfr_delay=dcfr_delay)
    res = sv.solve(rb, scal, evaluator if layout.num_model_leaves else None, cfr_plus=cfr_plus,
                   enforce_zero_sum=enforce_zero_sum, cfr_avg=cfr_avg, graph=graph)
    return res, trees, sv

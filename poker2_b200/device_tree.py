"""Public betting trees built on the GPU (`p2b_tree_count` / `p2b_tree_records`).

The device counterpart of `tree.build_trees` + `solver.device_layout`, i.e. of
`SparseCFREvaluator._construct_subgame` (p2/search/sparse_cfr_evaluator.py:141-306): the
records the solver kernel reads come out of one warp per subgame, no host-side tree is
built, and the only device-to-host transfer is one row of batch statistics.  The records
are byte-identical to those of the host builder (tested).
"""
from __future__ import annotations

import ctypes
from functools import cached_property

import numpy as np
import torch

from . import _lib
from . import tree as ptree


def pack_roots(roots: ptree.RoundState, bb=2) -> np.ndarray:
    """[B,16] int32 root records (the layout `p2b_tree_count` documents)."""
    n = roots.n
    out = np.zeros((n, 16), dtype=np.int32)
    cols = [roots.to_act, roots.pot, roots.stacks[:, 0], roots.stacks[:, 1], roots.committed[:, 0],
            roots.committed[:, 1], roots.min_raise, roots.actions_this_round,
            roots.is_allin[:, 0].astype(np.int64) + 2 * roots.is_allin[:, 1].astype(np.int64) + 4 * roots.done.astype(np.int64),
            roots.street, roots.button, roots.starting_stacks[:, 0], roots.starting_stacks[:, 1], roots.raises,
            np.broadcast_to(np.asarray(bb, dtype=np.int64), (n,))]
    for i, c in enumerate(cols):
        c = np.asarray(c, dtype=np.int64)
        if c.size and (c.min() < -(2 ** 31) or c.max() >= 2 ** 31):
            raise ValueError("chip counts must fit 32 bits")
        out[:, i] = c
    out[:, 15] = np.asarray(roots.scale, dtype=np.float32).view(np.int32)
    return out


class DeviceBuiltLayout:
    """The fields of `solver.DeviceTreeLayout`, held on the device; the numpy views are copied
    back only when something asks for them."""

    def __init__(self, *, subgames_dev, nodes_dev, to_level_major_dev, leaf_begin_dev, model_rows_dev, node_state_dev,
                 depth_offsets, max_internal, max_children, tree_depth, has_showdown, root_of_row_dev):
        self.subgames_dev, self.nodes_dev = subgames_dev, nodes_dev
        self.to_level_major_dev, self.leaf_begin_dev = to_level_major_dev, leaf_begin_dev
        self.model_rows_dev, self.node_state_dev = model_rows_dev, node_state_dev
        self.depth_offsets = depth_offsets
        self.max_internal, self.max_children, self.tree_depth = max_internal, max_children, tree_depth
        self.has_showdown = has_showdown
        self.root_of_row_dev = root_of_row_dev

    @property
    def rows(self) -> int:
        return int(self.nodes_dev.shape[0])

    @property
    def num_model_leaves(self) -> int:
        return int(self.model_rows_dev.shape[0])

    @cached_property
    def from_level_major_dev(self) -> torch.Tensor:
        inv = torch.empty_like(self.to_level_major_dev)
        inv[self.to_level_major_dev] = torch.arange(self.rows, device=inv.device, dtype=inv.dtype)
        return inv

    @cached_property
    def model_nodes_dev(self) -> torch.Tensor:
        return self.to_level_major_dev[self.model_rows_dev]

    # numpy views (device-to-host copies, made on first use)
    @cached_property
    def subgames(self) -> np.ndarray:
        from .solver import SUBGAME_DTYPE
        return self.subgames_dev.cpu().numpy().reshape(-1).view(SUBGAME_DTYPE)

    @cached_property
    def nodes(self) -> np.ndarray:
        from .solver import NODE_DTYPE
        return self.nodes_dev.cpu().numpy().reshape(-1).view(NODE_DTYPE)

    @cached_property
    def to_level_major(self) -> np.ndarray:
        return self.to_level_major_dev.cpu().numpy()

    @cached_property
    def from_level_major(self) -> np.ndarray:
        return self.from_level_major_dev.cpu().numpy()

    @cached_property
    def leaf_begin(self) -> np.ndarray:
        return self.leaf_begin_dev.cpu().numpy()

    @cached_property
    def model_rows(self) -> np.ndarray:
        return self.model_rows_dev.cpu().numpy()

    @cached_property
    def model_nodes(self) -> np.ndarray:
        return self.model_nodes_dev.cpu().numpy()

    def leaf_context(self) -> torch.Tensor:
        """[L,3] fp32 context of the model leaves (pot and both stacks as fractions of the two
        starting stacks together), computed on the device like `leaf_eval.leaf_context`."""
        if self.node_state_dev is None:
            raise ValueError("the layout was built without node_state=True")
        st = self.node_state_dev[self.model_rows_dev].to(torch.float32)
        total = (st[:, 3] + st[:, 4]).clamp(min=1.0)
        return torch.stack([st[:, 0] / total, st[:, 1] / total, st[:, 2] / total], dim=1).contiguous()


def build_device_layout(roots: ptree.RoundState, boards, bet_bins, max_depth: int, *, bb=2, max_raises=None,
                        device=None, node_state: bool = False) -> DeviceBuiltLayout:
    """Builds the solver's tree records for a batch of roots on `device`.  boards: [B,W] card
    ids (-1 = empty slot), numpy or tensor (host or device)."""
    device = torch.device(device if device is not None else "cuda:0")
    if device.type != "cuda":
        raise ValueError("build_device_layout requires a CUDA device.")
    B = roots.n
    if B == 0:
        raise ValueError("no subgames")
    bins = (ctypes.c_float * max(len(bet_bins), 1))(*[float(np.float32(b)) for b in bet_bins])
    n_bins, cap = len(bet_bins), -1 if max_raises is None else int(max_raises)
    D = int(max_depth)
    packed = torch.from_numpy(pack_roots(roots, bb)).to(device, non_blocking=True)
    if torch.is_tensor(boards):
        boards_dev = boards.to(device=device, dtype=torch.int64).contiguous()
    else:
        boards_dev = torch.from_numpy(np.ascontiguousarray(boards, dtype=np.int64)).to(device)
    i32 = dict(device=device, dtype=torch.int32)
    counts = torch.empty(B, 8, **i32)
    level_counts = torch.empty(B, D + 1, **i32)
    stream = _lib.stream_ptr(device)
    p = _lib.ptr
    with torch.cuda.device(device):
        _lib.call("p2b_tree_count", p(packed), B, bins, n_bins, D, cap, p(counts), p(level_counts), stream)
        # prefix sums over the subgames (plumbing): rows, model-leaf slots, level-major bases
        # (scans run along the contiguous dimension of transposed copies: torch's scan along the
        # outer dimension of a [B, few] tensor takes about a millisecond)
        c64 = counts.to(torch.int64)
        csum = torch.cumsum(c64[:, :3].t().contiguous(), dim=1).t()
        node_begin = (csum[:, 0] - c64[:, 0]).to(torch.int32)
        leaf_begin = (csum[:, 2] - c64[:, 2]).to(torch.int32)
        l64 = level_counts.to(torch.int64)
        level_tot = l64.sum(dim=0)
        depth_off = torch.cumsum(level_tot, dim=0) - level_tot
        level_base = (torch.cumsum(l64.t().contiguous(), dim=1).t() - l64 + depth_off[None, :]).contiguous()
        stats = torch.cat([csum[-1, :3], c64[:, 0].max()[None], c64[:, 1].max()[None], c64[:, 3].sum()[None],
                           c64[:, 4].max()[None], c64[:, 5].sum()[None], c64[:, 6].max()[None], level_tot]).cpu().numpy()
    rows, n_model = int(stats[0]), int(stats[2])
    if int(stats[7]) > 0:
        from .solver import MAX_NODES
        raise ValueError(f"a subgame has more than {MAX_NODES} nodes; the kernel supports up to {MAX_NODES}")
    if int(stats[6]) > 0:
        from .solver import MAX_CHILDREN
        if int(stats[6]) > MAX_CHILDREN:
            raise ValueError(f"at most {MAX_CHILDREN} actions per node are supported")
    tree_depth = int(stats[8])
    level_totals = stats[9:]
    depth_offsets = [0] + [int(x) for x in np.cumsum(level_totals[: tree_depth + 1])]
    subgames = torch.empty(B, 32, device=device, dtype=torch.uint8)
    nodes = torch.empty(rows, 16, device=device, dtype=torch.uint8)
    to_lm = torch.empty(rows, device=device, dtype=torch.int64)
    model_rows = torch.empty(n_model, device=device, dtype=torch.int64)
    state = torch.empty(rows, 8, **i32) if node_state else None
    with torch.cuda.device(device):
        _lib.call("p2b_tree_records", p(packed), p(boards_dev), int(boards_dev.shape[1]), B, bins, n_bins, D, cap,
                  p(node_begin), p(leaf_begin), p(level_base), p(subgames), p(nodes), p(to_lm),
                  p(model_rows) if n_model else None, p(state), stream)
        root_of_row = torch.repeat_interleave(torch.arange(B, device=device), c64[:, 0], output_size=rows)
    return DeviceBuiltLayout(subgames_dev=subgames, nodes_dev=nodes, to_level_major_dev=to_lm, leaf_begin_dev=leaf_begin,
                             model_rows_dev=model_rows, node_state_dev=state, depth_offsets=depth_offsets,
                             max_internal=int(stats[4]), max_children=int(stats[6]), tree_depth=tree_depth,
                             has_showdown=int(stats[5]) > 0, root_of_row_dev=root_of_row)

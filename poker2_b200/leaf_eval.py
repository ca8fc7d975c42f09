"""Leaf evaluators for subgames that end before the river: the callables a `SteppedSolver`
invokes between the two sweeps of every pass.

Upstream, the leaves at the start of the next street are valued by the value network
(`set_leaf_values`, p2/search/cfr_evaluator.py:1025-1047), and the value of such a
pre-chance state is the expectation over the next public card of the network's values on
the post-card beliefs (`ChanceNodeHelper.single_card_chance_values`,
p2/search/chance_node_helper.py:359-479).  `ChanceLeafEvaluator` computes that expectation
explicitly: the expansion over the next card and the per-leaf averaging are this library's
kernels (`chance.expand_next_card`, `chance.indexed_add_rows`); the network's GEMMs are
torch / cuBLAS.
"""
from __future__ import annotations

import numpy as np
import torch

from . import chance

NUM_HANDS = 1326


class ValueMLP(torch.nn.Module):
    """Value network stand-in with the shape of the benchmark configuration: input = two
    1326-combo ranges + 52-d board one-hot + 3 pot/stack scalars, `depth` hidden layers of
    `width` GELU units, output = 2 x 1326 hand values.  Random initialisation."""

    IN_FEATURES = 2 * NUM_HANDS + 52 + 3  # 2707
    IN_PADDED = 2720  # GEMM operands want rows that are multiples of 16 bytes; the extra columns are zero
    OUT_PADDED = 2656

    def __init__(self, width: int = 1536, depth: int = 4, *, dtype=torch.bfloat16, seed: int = 0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        dims = [self.IN_FEATURES] + [width] * depth + [2 * NUM_HANDS]
        padded = [self.IN_PADDED] + [width] * depth + [self.OUT_PADDED]
        layers = []
        for i in range(len(dims) - 1):
            lin = torch.nn.Linear(padded[i], padded[i + 1])
            with torch.no_grad():
                lin.weight.zero_()
                lin.weight[: dims[i + 1], : dims[i]] = torch.randn(dims[i + 1], dims[i], generator=g) / dims[i] ** 0.5
                lin.bias.zero_()
            layers.append(lin)
            if i < len(dims) - 2:
                layers.append(torch.nn.GELU())
        self.net = torch.nn.Sequential(*layers).to(dtype)
        self.dtype = dtype

    @torch.no_grad()
    def forward(self, beliefs: torch.Tensor, boards: torch.Tensor, context: torch.Tensor) -> torch.Tensor:
        """beliefs [S,2,1326] fp32, boards [S,L] int64 (-1 = empty), context [S,3] fp32
        -> values [S,2,1326] fp32."""
        S = beliefs.shape[0]
        x = torch.zeros(S, self.IN_PADDED, device=beliefs.device, dtype=self.dtype)
        x[:, : 2 * NUM_HANDS] = beliefs.reshape(S, 2 * NUM_HANDS)
        onehot = torch.zeros(S, 53, device=beliefs.device, dtype=self.dtype)
        onehot.scatter_(1, torch.where(boards >= 0, boards, torch.full_like(boards, 52)), 1.0)
        x[:, 2 * NUM_HANDS: 2 * NUM_HANDS + 52] = onehot[:, :52]
        x[:, 2 * NUM_HANDS + 52: self.IN_FEATURES] = context
        y = self.net(x)[:, : 2 * NUM_HANDS]
        return y.to(torch.float32).view(S, 2, NUM_HANDS)


def leaf_context(trees, node_index) -> torch.Tensor:
    """[L,3] fp32 context of the tree nodes `node_index` (upstream numbering): pot and both
    stacks as fractions of the two starting stacks together."""
    st = trees.state
    idx = np.asarray(node_index, dtype=np.int64)
    total = np.maximum(st.starting_stacks[idx].astype(np.float32).sum(axis=1), np.float32(1.0))
    f32 = lambda a: a.astype(np.float32)  # noqa: E731  (fp32 division, as the upstream encoder does)
    ctx = np.stack([f32(st.pot[idx]) / total, f32(st.stacks[idx, 0]) / total, f32(st.stacks[idx, 1]) / total], axis=1)
    return torch.from_numpy(np.ascontiguousarray(ctx, dtype=np.float32))


class ChanceLeafEvaluator:
    """values(leaf) = mean over the next public card of model(post-card beliefs).

    boards: [L,W] int64 public cards of each leaf with -1 in the empty slots (at least one);
    context: [L,3] fp32; model(beliefs [S,2,1326], boards [S,W], context [S,3]) -> [S,2,1326].
    Leaves are processed `chunk` at a time (a chunk expands to about 48 x chunk samples)."""

    def __init__(self, model, boards: torch.Tensor, context: torch.Tensor, device: torch.device, *, chunk: int = 2048):
        self.model = model
        self.boards = boards.to(device=device, dtype=torch.int64).contiguous()
        self.context = context.to(device=device, dtype=torch.float32).contiguous()
        self.chunk = int(chunk)
        self.samples_per_call = int((52 - (self.boards >= 0).sum(dim=1)).sum().item())
        self.calls = 0
        # a bf16 `ValueMLP` takes the fused path: the network input is written directly by the
        # expansion kernel and its bf16 output is averaged per leaf without an fp32 copy
        self.fused = isinstance(model, ValueMLP) and model.dtype == torch.bfloat16
        self._chunks = []
        for a in range(0, self.boards.shape[0], self.chunk):
            b = min(a + self.chunk, self.boards.shape[0])
            off = chance.sample_offsets_of(self.boards[a:b])
            self._chunks.append((a, b, off, int(off[-1].item())))

    def _call_fused(self, leaf_beliefs: torch.Tensor) -> torch.Tensor:
        L, W = leaf_beliefs.shape[0], leaf_beliefs.shape[2]
        out = torch.zeros(L, 2, W, device=leaf_beliefs.device, dtype=torch.float32)
        for a, b, off, n_samples in self._chunks:
            x = chance.expand_features_bf16(leaf_beliefs[a:b], self.boards[a:b], off, n_samples, self.context[a:b],
                                            self.model.IN_PADDED)
            y = self.model.net(x)
            chance.indexed_mean_bf16(y, off, out[a:b])
        self.calls += 1
        return out

    def __call__(self, leaf_beliefs: torch.Tensor) -> torch.Tensor:
        if self.fused:
            return self._call_fused(leaf_beliefs)
        L = leaf_beliefs.shape[0]
        out = torch.empty(L, 2, NUM_HANDS, device=leaf_beliefs.device, dtype=torch.float32)
        for a in range(0, L, self.chunk):
            b = min(a + self.chunk, L)
            pre = leaf_beliefs[a:b, :, :NUM_HANDS].contiguous()
            ctx = self.context[a:b]
            out[a:b] = chance.single_card_chance_values(
                pre, self.boards[a:b], lambda post, samples, lookup: self.model(post, samples, ctx[lookup]))
        self.calls += 1
        return out


class DirectLeafEvaluator:
    """values(leaf) = model(beliefs at the leaf): the network is trained to predict the
    pre-chance value itself, which is how the upstream CFR loop calls it."""

    def __init__(self, model, boards: torch.Tensor, context: torch.Tensor, device: torch.device):
        self.model = model
        self.boards = boards.to(device=device, dtype=torch.int64).contiguous()
        self.context = context.to(device=device, dtype=torch.float32).contiguous()

    def __call__(self, leaf_beliefs: torch.Tensor) -> torch.Tensor:
        return self.model(leaf_beliefs[..., :NUM_HANDS].contiguous(), self.boards, self.context)

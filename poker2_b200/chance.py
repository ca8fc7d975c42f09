"""Chance-node helpers on the GPU: the counterpart of
`ChanceNodeHelper.single_card_chance_values` (p2/search/chance_node_helper.py:359-479).

`expand_next_card` enumerates, for every root, the boards with one more public card and
the re-blocked, re-normalised beliefs on each; `indexed_add_rows` is the ordered
index_add_ / mean that folds the leaf-model values of the samples back onto their roots.
`single_card_chance_values` composes the two around a caller-supplied value function (the
leaf model: its GEMMs stay in torch / cuBLAS).
"""
from __future__ import annotations

from typing import Callable

import torch

from . import _lib

NUM_HANDS = _lib.NUM_HANDS


def expand_next_card(pre_beliefs: torch.Tensor, boards: torch.Tensor):
    """pre_beliefs [B,2,1326] fp32, boards [B,L] int64 (-1 = empty slot, at least one empty)
    -> (post_beliefs [S,2,1326], root_lookup [S] int64, board_samples [S,L] int64) with
    S = sum over roots of the number of cards not on the board."""
    _lib.require_cuda(pre_beliefs, "expand_next_card")
    assert pre_beliefs.dim() == 3 and tuple(pre_beliefs.shape[1:]) == (2, NUM_HANDS)
    assert pre_beliefs.dtype == torch.float32 and pre_beliefs.is_contiguous()
    boards = boards.to(device=pre_beliefs.device, dtype=torch.int64).contiguous()
    B, L = boards.shape
    assert B == pre_beliefs.shape[0]
    free = 52 - (boards >= 0).sum(dim=1)
    offsets = torch.zeros(B + 1, dtype=torch.int64, device=boards.device)
    offsets[1:] = torch.cumsum(free, dim=0)
    S = int(offsets[-1].item())
    post = torch.empty(S, 2, NUM_HANDS, device=boards.device, dtype=torch.float32)
    lookup = torch.empty(S, dtype=torch.int64, device=boards.device)
    samples = torch.empty(S, L, dtype=torch.int64, device=boards.device)
    with torch.cuda.device(boards.device):
        _lib.call("p2b_chance_expand", _lib.ptr(pre_beliefs), _lib.ptr(boards), L, _lib.ptr(offsets), B, S,
                  _lib.ptr(post), _lib.ptr(lookup), _lib.ptr(samples), _lib.stream_ptr(boards.device))
    return post, lookup, samples


def indexed_add_rows(out: torch.Tensor, index: torch.Tensor, src: torch.Tensor, *, mean: bool = False,
                     accumulate: bool = True) -> torch.Tensor:
    """out[index[i]] += src[i] for a SORTED int64 index, added in ascending i (deterministic,
    same order as a CPU index_add_).  `mean` divides each row by max(count, 1);
    `accumulate=False` overwrites `out`."""
    _lib.require_cuda(out, "indexed_add_rows")
    assert out.is_contiguous() and src.is_contiguous() and index.is_contiguous()
    assert out.dtype == torch.float32 == src.dtype and index.dtype == torch.int64
    assert src.shape[0] == index.shape[0] and src.shape[1:] == out.shape[1:]
    width = out[0].numel() if out.shape[0] else 0
    with torch.cuda.device(out.device):
        _lib.call("p2b_indexed_add_rows", _lib.ptr(out), _lib.ptr(index), _lib.ptr(src), src.shape[0], out.shape[0],
                  width, int(mean), int(accumulate), _lib.stream_ptr(out.device))
    return out


def single_card_chance_values(pre_beliefs: torch.Tensor, boards: torch.Tensor,
                              value_fn: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor]):
    """Expected leaf values over the next public card: `value_fn(post_beliefs, board_samples,
    root_lookup) -> [S,2,1326]` is evaluated on every (root, card) sample and averaged per
    root (chance_node_helper.py:359-479)."""
    post, lookup, samples = expand_next_card(pre_beliefs, boards)
    values = value_fn(post, samples, lookup).to(torch.float32).contiguous()
    out = torch.empty(pre_beliefs.shape[0], 2, NUM_HANDS, device=pre_beliefs.device, dtype=torch.float32)
    return indexed_add_rows(out, lookup, values, mean=True, accumulate=False)


def sample_offsets_of(boards: torch.Tensor) -> torch.Tensor:
    """[B+1] int64 exclusive prefix of the number of cards not on each board."""
    free = 52 - (boards >= 0).sum(dim=1)
    offsets = torch.zeros(boards.shape[0] + 1, dtype=torch.int64, device=boards.device)
    offsets[1:] = torch.cumsum(free, dim=0)
    return offsets


def expand_features_bf16(pre_beliefs: torch.Tensor, boards: torch.Tensor, offsets: torch.Tensor, num_samples: int,
                         context: torch.Tensor, feature_stride: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """Network input rows [S, feature_stride] bf16 for every (root, next card) sample: the fused
    form of `expand_next_card` + cast + board one-hot + context.  pre_beliefs [B,2,W] fp32 with
    W = 1326 or the padded 1344 (any last-dimension stride of 1)."""
    _lib.require_cuda(pre_beliefs, "expand_features_bf16")
    B = pre_beliefs.shape[0]
    assert pre_beliefs.dtype == torch.float32 and pre_beliefs.stride(2) == 1 and pre_beliefs.stride(0) == 2 * pre_beliefs.stride(1)
    assert boards.dtype == torch.int64 and boards.is_contiguous() and boards.shape[0] == B
    assert context.dtype == torch.float32 and context.is_contiguous() and tuple(context.shape) == (B, 3)
    if out is None:
        out = torch.empty(num_samples, feature_stride, device=pre_beliefs.device, dtype=torch.bfloat16)
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and tuple(out.shape) == (num_samples, feature_stride)
    with torch.cuda.device(pre_beliefs.device):
        _lib.call("p2b_chance_expand_features", _lib.ptr(pre_beliefs), pre_beliefs.stride(1), _lib.ptr(boards),
                  boards.shape[1], _lib.ptr(offsets), B, num_samples, _lib.ptr(context), _lib.ptr(out), feature_stride,
                  None, _lib.stream_ptr(pre_beliefs.device))
    return out


def indexed_mean_bf16(src: torch.Tensor, offsets: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r, p, :1326] = fp32 mean over the samples offsets[r]..offsets[r+1] of src[sample, p*1326:(p+1)*1326]
    (bf16 rows); out is [B,2,W] fp32 with W >= 1326."""
    _lib.require_cuda(src, "indexed_mean_bf16")
    assert src.dtype == torch.bfloat16 and src.stride(1) == 1 and out.dtype == torch.float32
    assert out.stride(2) == 1 and out.stride(0) == 2 * out.stride(1)
    with torch.cuda.device(src.device):
        _lib.call("p2b_indexed_mean_bf16", _lib.ptr(src), src.stride(0), _lib.ptr(offsets), out.shape[0], _lib.ptr(out),
                  out.stride(1), _lib.stream_ptr(src.device))
    return out

"""7-card hand evaluation on sm_100a: same entry points, argument meaning and error
behaviour as the upstream module p2/env/rules_triton.py, backed by hand-written CUDA.

The upstream names (`*_triton`) are kept as aliases so that an import swap is enough:
    import poker2_b200.rules as rules_triton
"""
from __future__ import annotations

import torch

from . import _lib

NUM_HANDS = _lib.NUM_HANDS


def backend_is_available() -> bool:
    """Counterpart of `triton_is_available` (rules_triton.py:19): True when the compiled
    kernel library is present."""
    return _lib.library_available()


def _require_backend() -> None:
    if not backend_is_available():
        raise RuntimeError(
            "libpoker2_b200.so is not built. Run `python -m poker2_b200.build` in a CUDA "
            "environment to use the CUDA hand evaluator."
        )


def compare_7_single_batch(ab_batch: torch.Tensor) -> torch.Tensor:
    """[N,2,4,13] one-hot planes -> int32 [N] in {1,-1,0} (rules_triton.py:36-51)."""
    _require_backend()
    if ab_batch.dim() != 4 or tuple(ab_batch.shape[1:]) != (2, 4, 13):
        raise ValueError(f"Expected [N, 2, 4, 13] input, got {tuple(ab_batch.shape)}")
    _lib.require_cuda(ab_batch, "CUDA hand evaluator")
    planes = ab_batch.contiguous().to(torch.int8)
    out = torch.empty((planes.shape[0],), device=planes.device, dtype=torch.int32)
    with torch.cuda.device(planes.device):
        _lib.call("p2b_compare7_planes", _lib.ptr(planes), planes.shape[0], _lib.ptr(out),
                  _lib.stream_ptr(planes.device))
    return out


def compare_7_batches(a_batch: torch.Tensor, b_batch: torch.Tensor) -> torch.Tensor:
    """Two [N,4,13] plane batches -> int32 [N] (rules_triton.py:54-60)."""
    if a_batch.shape != b_batch.shape:
        raise ValueError("a_batch and b_batch must have the same shape.")
    if a_batch.dim() != 3 or tuple(a_batch.shape[1:]) != (4, 13):
        raise ValueError(f"Expected [N, 4, 13] inputs, got {tuple(a_batch.shape)}")
    return compare_7_single_batch(torch.stack([a_batch, b_batch], dim=1).bool())


def _as_i16(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.int16 and t.is_contiguous():
        return t
    return t.contiguous().to(torch.int16)


def compare_7_cards_single_batch(cards_batch: torch.Tensor) -> torch.Tensor:
    """[N,2,7] card ids 0..51 -> int32 [N] in {1,-1,0} (rules_triton.py:78-93)."""
    _require_backend()
    if cards_batch.dim() != 3 or tuple(cards_batch.shape[1:]) != (2, 7):
        raise ValueError(f"Expected [N, 2, 7] input, got {tuple(cards_batch.shape)}")
    _lib.require_cuda(cards_batch, "CUDA hand evaluator")
    cards = _as_i16(cards_batch)
    out = torch.empty((cards.shape[0],), device=cards.device, dtype=torch.int32)
    with torch.cuda.device(cards.device):
        _lib.call("p2b_compare7_cards", _lib.ptr(cards), cards.shape[0], _lib.ptr(out),
                  _lib.stream_ptr(cards.device))
    return out


def rank_7_cards_single_batch(cards_batch: torch.Tensor) -> torch.Tensor:
    """[N,7] card ids -> int32 [N] packed scores, higher = stronger
    (rules_triton.py:96-117)."""
    _require_backend()
    if cards_batch.dim() != 2 or cards_batch.shape[1] != 7:
        raise ValueError(f"Expected [N, 7] input, got {tuple(cards_batch.shape)}")
    _lib.require_cuda(cards_batch, "CUDA hand evaluator")
    cards = _as_i16(cards_batch)
    out = torch.empty((cards.shape[0],), device=cards.device, dtype=torch.int32)
    with torch.cuda.device(cards.device):
        _lib.call("p2b_rank7_cards", _lib.ptr(cards), cards.shape[0], _lib.ptr(out),
                  _lib.stream_ptr(cards.device))
    return out


def rank_hands(board: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """[M,5] board card ids -> (int32 [M,1326] packed score per combo, int64 [M,1326]
    stable ascending argsort), the drop-in for `rank_hands` (rules_triton.py:120-148)."""
    _require_backend()
    if board.dim() != 2 or board.shape[1] != 5:
        raise ValueError(f"board must be [M, 5], got {tuple(board.shape)}")
    _lib.require_cuda(board, "CUDA hand evaluator")
    b16 = _as_i16(board)
    m = b16.shape[0]
    scores = torch.empty((m, NUM_HANDS), device=board.device, dtype=torch.int32)
    order = torch.empty((m, NUM_HANDS), device=board.device, dtype=torch.int64)
    with torch.cuda.device(board.device):
        _lib.call("p2b_rank_hands", _lib.ptr(b16), m, _lib.ptr(scores), _lib.ptr(order), None,
                  _lib.stream_ptr(board.device))
    return scores, order


# upstream spellings
triton_is_available = backend_is_available
compare_7_single_batch_triton = compare_7_single_batch
compare_7_batches_triton = compare_7_batches
compare_7_cards_single_batch_triton = compare_7_cards_single_batch
rank_7_cards_single_batch_triton = rank_7_cards_single_batch
rank_hands_triton = rank_hands

"""Blocker-aware river showdown values on sm_100a.

Counterpart of `CFREvaluator._init_hand_rank_data` and `_showdown_value_both`
(p2/search/cfr_evaluator.py:406-601).  Board tables are built once per distinct board and
shared by every showdown node of that board.
"""
from __future__ import annotations

import torch

from . import _lib

NUM_HANDS = _lib.NUM_HANDS


class BoardTables:
    """Per-board strength order, tie groups and per-card hand lists, resident on the GPU."""

    def __init__(self, boards: torch.Tensor):
        if boards.dim() != 2 or boards.shape[1] != 5:
            raise ValueError(f"boards must be [M, 5], got {tuple(boards.shape)}")
        _lib.require_cuda(boards, "BoardTables")
        self.device = boards.device
        self.num_boards = boards.shape[0]
        b16 = boards.contiguous().to(torch.int16)
        self.blob = torch.empty((self.num_boards, _lib.TABLE_BYTES), device=self.device, dtype=torch.uint8)
        with torch.cuda.device(self.device):
            _lib.call("p2b_rank_hands", _lib.ptr(b16), self.num_boards, None, None, _lib.ptr(self.blob),
                      _lib.stream_ptr(self.device))


def showdown_values(
    tables: BoardTables,
    beliefs: torch.Tensor,
    potential: torch.Tensor,
    scale: torch.Tensor,
    table_of_row: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """beliefs [R,2,1326] fp32, potential [R,2] int64, scale [R] fp32 -> values [R,2,1326]:
    values[r,p] = showdown EV of player p's hands against beliefs[r,1-p], times
    potential[r,p]/scale[r].  Row r uses board table `table_of_row[r]` (default r)."""
    _lib.require_cuda(beliefs, "showdown_values")
    if beliefs.dim() != 3 or tuple(beliefs.shape[1:]) != (2, NUM_HANDS):
        raise ValueError(f"beliefs must be [R, 2, {NUM_HANDS}], got {tuple(beliefs.shape)}")
    rows = beliefs.shape[0]
    assert beliefs.dtype == torch.float32 and beliefs.is_contiguous()
    potential = potential.to(device=beliefs.device, dtype=torch.int64).contiguous()
    scale = scale.to(device=beliefs.device, dtype=torch.float32).contiguous()
    assert tuple(potential.shape) == (rows, 2) and tuple(scale.shape) == (rows,)
    if table_of_row is not None:
        table_of_row = table_of_row.to(device=beliefs.device, dtype=torch.int32).contiguous()
        assert tuple(table_of_row.shape) == (rows,)
    elif rows != tables.num_boards:
        raise ValueError("table_of_row is required when rows != number of boards")
    if out is None:
        out = torch.empty_like(beliefs)
    assert out.is_contiguous() and out.shape == beliefs.shape and out.dtype == torch.float32
    with torch.cuda.device(beliefs.device):
        _lib.call("p2b_showdown_values", _lib.ptr(tables.blob), _lib.ptr(table_of_row), _lib.ptr(beliefs),
                  2 * NUM_HANDS, _lib.ptr(potential), _lib.ptr(scale), _lib.ptr(out), 2 * NUM_HANDS, rows,
                  _lib.stream_ptr(beliefs.device))
    return out

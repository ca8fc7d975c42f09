"""ctypes front of the C hand-rank oracle (oracle/rank7.c).  Test infrastructure only."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libp2oracle.so")
_lib = None

MODE_PLANES = 0  # a repeated card id counts once (p2/env/rules.py:87-102)
MODE_IDS = 1  # rank multiplicity counts repeats (p2/env/rules_triton.py:431-446)


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "rank7.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "_build/libp2oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(_LIB_PATH)
        p16 = ctypes.POINTER(ctypes.c_int16)
        p32 = ctypes.POINTER(ctypes.c_int32)
        lib.p2o_rank7_batch.argtypes = [p16, ctypes.c_int64, ctypes.c_int, p32]
        lib.p2o_rank_boards.argtypes = [p16, ctypes.c_int64, ctypes.c_int, p32]
        lib.p2o_compare7_batch.argtypes = [p16, ctypes.c_int64, ctypes.c_int, p32]
        lib.p2o_rank_planes.argtypes = [ctypes.POINTER(ctypes.c_int8), ctypes.c_int64, p32]
        lib.p2o_rank_planes.restype = None
        lib.p2o_rank7_batch.restype = None
        lib.p2o_rank_boards.restype = None
        lib.p2o_compare7_batch.restype = None
        _lib = lib
    return _lib


def _p(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


def rank7(hands: np.ndarray, mode: int = MODE_IDS) -> np.ndarray:
    """hands [N,7] ints -> packed scores [N] int32."""
    h = np.ascontiguousarray(hands, dtype=np.int16)
    assert h.ndim == 2 and h.shape[1] == 7
    out = np.empty(h.shape[0], dtype=np.int32)
    _load().p2o_rank7_batch(_p(h, ctypes.c_int16), h.shape[0], mode, _p(out, ctypes.c_int32))
    return out


def rank_boards(boards: np.ndarray, mode: int = MODE_IDS) -> np.ndarray:
    """boards [M,5] -> packed scores of all combos [M,1326] int32."""
    b = np.ascontiguousarray(boards, dtype=np.int16)
    assert b.ndim == 2 and b.shape[1] == 5
    out = np.empty((b.shape[0], 1326), dtype=np.int32)
    _load().p2o_rank_boards(_p(b, ctypes.c_int16), b.shape[0], mode, _p(out, ctypes.c_int32))
    return out


def compare7(cards: np.ndarray, mode: int = MODE_IDS) -> np.ndarray:
    """cards [N,2,7] -> sign of (score(a) - score(b)) [N] int32."""
    c = np.ascontiguousarray(cards, dtype=np.int16)
    assert c.ndim == 3 and c.shape[1:] == (2, 7)
    out = np.empty(c.shape[0], dtype=np.int32)
    _load().p2o_compare7_batch(_p(c, ctypes.c_int16), c.shape[0], mode, _p(out, ctypes.c_int32))
    return out


def rank_planes(planes: np.ndarray) -> np.ndarray:
    """planes [N,4,13] (non-zero = card present) -> packed scores [N] int32 of the card sets."""
    p = np.ascontiguousarray(planes != 0, dtype=np.int8)
    assert p.ndim == 3 and p.shape[1:] == (4, 13)
    out = np.empty(p.shape[0], dtype=np.int32)
    _load().p2o_rank_planes(_p(p, ctypes.c_int8), p.shape[0], _p(out, ctypes.c_int32))
    return out


def compare_planes(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Sign of score(a) - score(b) for two [N,4,13] plane batches (rules.py:412-426)."""
    sa, sb = rank_planes(a).astype(np.int64), rank_planes(b).astype(np.int64)
    return np.sign(sa - sb).astype(np.int32)


def rank_hands(boards: np.ndarray, mode: int = MODE_IDS):
    """Per-board scores plus the stable ascending argsort, as the upstream
    `rank_hands_triton` returns them (p2/env/rules_triton.py:120-148)."""
    scores = rank_boards(boards, mode)
    order = np.argsort(scores, axis=1, kind="stable").astype(np.int64)
    return scores, order

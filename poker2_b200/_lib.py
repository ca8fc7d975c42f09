"""ctypes binding of libpoker2_b200.so (the C ABI declared in include/poker2_b200.h).

There is no CPU fallback: if the shared library is missing or a call fails, an exception
is raised.
"""
from __future__ import annotations

import ctypes
import os

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libpoker2_b200.so")
TABLE_BYTES = 18592
NUM_HANDS = 1326

_lib = None

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int
_f32 = ctypes.c_float

# name -> argtypes; every function returns int
_SIGNATURES = {
    "p2b_rank7_cards": [_vp, _i64, _vp, _vp],
    "p2b_compare7_cards": [_vp, _i64, _vp, _vp],
    "p2b_compare7_planes": [_vp, _i64, _vp, _vp],
    "p2b_rank_hands": [_vp, _i64, _vp, _vp, _vp, _vp],
    "p2b_showdown_values": [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _i64, _vp],
    "p2b_showdown_ev_sorted": [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _vp, _vp],
    "p2b_cfr_solve": [_vp, _vp, _i32, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64,
                      _vp, _i32, _i32, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _f32, _vp],
    "p2b_cfr_step": [_vp, _vp, _i32, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64,
                     _vp, _i32, _i32, _i32, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp,
                     _vp, _vp, _vp],
    "p2b_cfr_warm_seed": [_vp, _i64, _vp, _f32, _vp, _vp, _vp],
    "p2b_cfr_noalloc_status": [_vp, _vp],
    "p2b_cfr_iteration_timing": [_i32],
    "p2b_cfr_iteration_ms": [_vp],
    "p2b_cfr_solve_noalloc": [_vp, _vp, _i32, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                              _i32, _i32, _i32, _vp],
    "p2b_step_dcfr_update": [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _vp],
    "p2b_step_block_normalize": [_vp, _vp, _vp, _i64, _i32, _i32, _f32, _vp],
    "p2b_step_regret_matching_divide": [_vp, _vp, _vp, _vp, _i64, _f32, _vp],
    "p2b_step_weight_child_values": [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _vp],
    "p2b_step_update_average_values": [_vp, _vp, _vp, _vp, _vp, _i64, _vp],
    "p2b_step_mix_zero_sum": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp],
    "p2b_step_scaled_difference": [_vp, _vp, _vp, _vp, _vp, _i64, _vp],
    "p2b_step_regret_tail": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _vp],
    "p2b_step_average_policy_mix": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _f32, _vp],
    "p2b_step_parent_sum": [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i64, _vp],
    "p2b_step_divide_by_parent_sum": [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _vp],
    "p2b_step_unblocked_mass": [_vp, _vp, _vp, _i64, _vp],
    "p2b_step_unblocked_mass_ratio": [_vp, _vp, _vp, _vp, _i64, _f32, _vp],
    "p2b_step_weighted_parent_sum": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _vp],
    "p2b_step_reach_weights": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _vp],
    "p2b_step_deep_beliefs": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _f32, _vp],
    "p2b_chance_expand": [_vp, _vp, _i32, _vp, _i64, _i64, _vp, _vp, _vp, _vp],
    "p2b_indexed_add_rows": [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp],
    "p2b_chance_expand_features": [_vp, _i64, _vp, _i32, _vp, _i64, _i64, _vp, _vp, _i64, _vp, _vp],
    "p2b_indexed_mean_bf16": [_vp, _i64, _vp, _i64, _vp, _i64, _vp],
    "p2b_expand_on_boards": [_vp, _i64, _vp, _i32, _i64, _i64, _vp, _vp],
    "p2b_mean_over_hand_perms": [_vp, _vp, _i32, _i64, _vp, _vp],
    "p2b_tree_count": [_vp, _i32, _vp, _i32, _i32, _i32, _vp, _vp, _vp],
    "p2b_tree_records": [_vp, _vp, _i32, _i32, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "p2b_selftest_division": [ctypes.c_uint64, ctypes.c_uint32, _vp, _vp, _vp],
    "p2b_selftest_division_sweep": [_vp, _vp, _vp],
}
# functions whose return value is a quantity, not a status code
_VALUE_FUNCS = {"p2b_cfr_scratch_floats": ([_i32, _i32], _i64), "p2b_cfr_default_blocks": ([], _i32),
                "p2b_cfr_solve_scratch_floats": ([_i32, _i32, _i32, _i32, _i64], _i64),
                "p2b_cfr_noalloc_scratch_floats": ([], _i64), "p2b_cfr_path_policy": ([_i32], _i32)}


def library_available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    """Loads the shared library once; raises RuntimeError if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m poker2_b200.build` "
                "(poker2_b200 has no CPU or PyTorch fallback)"
            )
        handle = ctypes.CDLL(LIB_PATH)
        handle.p2b_last_error.restype = ctypes.c_char_p
        handle.p2b_last_error.argtypes = []
        handle.p2b_version.restype = ctypes.c_int
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = ctypes.c_int
        for name, (argtypes, restype) in _VALUE_FUNCS.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = handle
    return _lib


def exported_symbols():
    return ["p2b_last_error", "p2b_version", *_SIGNATURES.keys(), *_VALUE_FUNCS.keys()]


def call(name: str, *args) -> None:
    handle = lib()
    rc = getattr(handle, name)(*args)
    if rc != 0:
        msg = handle.p2b_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{name} failed ({rc}): {msg}")


def ptr(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_ptr(device: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(t: torch.Tensor, what: str) -> None:
    if t.device.type != "cuda":
        raise ValueError(f"{what} requires a CUDA tensor.")

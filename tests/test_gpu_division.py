"""The solver's shared-divisor division must round exactly like IEEE fp32 division."""
import pytest
import torch

from poker2_b200 import _lib

pytestmark = pytest.mark.gpu


def test_shared_divisor_division_is_ieee_exact(cuda_device):
    counts = torch.zeros(2, dtype=torch.int64, device=cuda_device)
    pairs = 1 << 32
    for seed in (1, 2, 3):
        _lib.call("p2b_selftest_division", pairs, seed, _lib.ptr(counts[0:]), _lib.ptr(counts[1:]),
                  _lib.stream_ptr(cuda_device))
    torch.cuda.synchronize()
    mismatches, short_path = (int(v) for v in counts.tolist())
    assert mismatches == 0
    # the comparison is only meaningful if most pairs really took the short sequence
    assert short_path > 3 * pairs // 2


def test_division_sweep_over_all_divisor_mantissas(cuda_device):
    """Every divisor mantissa at five exponents against numerators on rounding boundaries: the short
    sequence fails, if at all, on rare divisor mantissas that random draws would almost never hit."""
    counts = torch.zeros(2, dtype=torch.int64, device=cuda_device)
    _lib.call("p2b_selftest_division_sweep", _lib.ptr(counts[0:]), _lib.ptr(counts[1:]), _lib.stream_ptr(cuda_device))
    torch.cuda.synchronize()
    mismatches, checked = (int(v) for v in counts.tolist())
    assert checked == (1 << 23) * 5 * 16
    assert mismatches == 0

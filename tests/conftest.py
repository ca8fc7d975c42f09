import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from poker2_b200 import build

    build.build()
    # The fixtures are batches of a few subgames, which the default policy would hand to the general kernel;
    # the suite wants the lean iteration kernel on them too (tests/test_gpu_path_policy.py covers the default).
    from poker2_b200 import solver

    solver.set_path_policy("lean")
    return torch.device("cuda:0")

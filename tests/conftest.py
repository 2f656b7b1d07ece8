import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def cuda_lib():
    """The in-tree sm_100a library; GPU tests fail (not skip) when it is missing."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from causal_trainer_dev_b200.ops import lib

    lib.require_gpu_lib()
    return lib

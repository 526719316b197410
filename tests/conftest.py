import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a real B200 (run with `pytest -m gpu`)")
    config.addinivalue_line("markers", "slow: multi-process / long-running CPU test")


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from llmctl_b200.ops import native
    native.lib()  # fail loudly if the extension is missing on a GPU box
    return torch.device("cuda", 0)

import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(ROOT / "tests" / "golden" / "gguf_golden.npz")


@pytest.fixture(scope="session")
def cuda():
    """The CUDA device for GPU tests; importing the package must load the native module."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import torch_ggml_ops_b200  # noqa: F401  (fails loudly if the extension is missing)

    return torch.device("cuda:0")

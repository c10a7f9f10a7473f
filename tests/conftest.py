import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests" / "golden"))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with `-m gpu`")


@pytest.fixture(scope="session")
def lib_path():
    """The in-tree shared library; built here when nvcc is present and the file is missing or stale."""
    from logo_b200 import build

    try:
        return build.build()
    except RuntimeError as exc:
        if build.LIB_PATH.exists():   # no nvcc on this machine: use the prebuilt file
            return build.LIB_PATH
        pytest.skip(f"liblogo_b200.so is neither built nor buildable here: {exc}")


@pytest.fixture(scope="session")
def golden():
    return {p.stem: np.load(p) for p in GOLDEN.glob("*.npz")}


@pytest.fixture(scope="session")
def cuda_device(lib_path):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")

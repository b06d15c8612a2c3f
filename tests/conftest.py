import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


def load_fixture(name: str) -> dict:
    """Loads tests/golden/<name>.npz as torch tensors (bf16 is stored as uint16 bit patterns)."""
    out = {}
    with np.load(GOLDEN / f"{name}.npz") as z:
        for key in z.files:
            a = z[key]
            if a.dtype == np.uint16:
                out[key] = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
            elif a.ndim == 0:
                out[key] = a.item()
            else:
                out[key] = torch.from_numpy(a.copy())
    return out


def fixture_names(prefix: str):
    return sorted(p.stem for p in GOLDEN.glob(f"{prefix}*.npz"))


@pytest.fixture(scope="session")
def built_libs():
    """Builds (if needed) and loads the shared libraries once per session."""
    from diopi_b200 import _lib, build

    build.build()
    return _lib.load()

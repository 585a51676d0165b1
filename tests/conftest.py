import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on a B200")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _reset_global_state():
    """The reference's autouse fixture (tests/conftest.py:6-9): precision flag off, seeds fixed.  The
    default device is left alone so CPU-side oracle tensors stay on the CPU."""
    from triturus_b200.utils import set_tf32_enabled

    set_tf32_enabled(False)
    torch.manual_seed(42)
    np.random.seed(42)
    yield
    set_tf32_enabled(False)


def load_golden(name: str) -> dict:
    with np.load(GOLDEN / f"{name}.npz") as z:
        return {k: torch.from_numpy(z[k].copy()) for k in z.files}


LM_GOLDEN = ["lm_reftest", "lm_cfg1", "lm_cfg2", "lm_cfg3", "lm_neginf", "lm_single"]
LT_GOLDEN = ["lt_reftest", "lt_cfg4", "lt_cfg5", "lt_neginf"]

# Tolerances in log space against the float64 evaluation (absolute), by precision mode.
ATOL = {"tf32": 2e-3, "3xtf32": 1e-4}

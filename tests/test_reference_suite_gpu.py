"""The reference's own hot-path tests (tests/lm2exp.py:10-23, tests/lt2exp.py:14-40), restated against the
drop-in import paths `triturus.lm2exp`, `triturus.lt2exp`, `triturus.utils`: same shapes, same input
distributions, same torch.allclose tolerances (default rtol 1e-5 / atol 1e-8 with TF32 off, rtol 5e-4 with
TF32 on).  The ground truth is the oracle's fp32 restatement of the reference's torch baseline, evaluated
on the GPU so that, as in the reference, it runs on the same device as the kernel."""

import itertools

import pytest
import torch

from oracle.logspace_oracle import lm2exp_fp32 as torch_lm2exp
from oracle.logspace_oracle import lt2exp_fp32 as torch_lt2exp
from triturus.lm2exp import lm2exp
from triturus.lt2exp import lt2exp
from triturus.utils import ensure_reproducibility, set_tf32_enabled

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _reference_global_state():
    set_tf32_enabled(False)
    ensure_reproducibility(determinism=True, device="cuda")
    yield
    set_tf32_enabled(False)
    torch.set_default_device("cpu")
    torch.use_deterministic_algorithms(False)


@pytest.mark.parametrize("allow_tf32", [False, True])
def test_lm2exp(allow_tf32: bool):
    set_tf32_enabled(allow_tf32)
    batch, m, k, n = 24, 150, 100, 200
    a = torch.rand(batch, m, k)
    b = torch.randn(batch, k, n)
    set_tf32_enabled(False)  # ground truth in full fp32
    gt = torch_lm2exp(a, b)
    set_tf32_enabled(allow_tf32)
    c = lm2exp(a, b)
    if allow_tf32:
        assert torch.allclose(gt, c, rtol=5e-4)
    else:
        assert torch.allclose(gt, c)


@pytest.mark.parametrize("mode,allow_tf32", list(itertools.product(["auto", "split", "unsplit"], [False, True])))
def test_lt2exp(mode: str, allow_tf32: bool):
    set_tf32_enabled(allow_tf32)
    batch, m, j, k, n = 3, 75, 50, 50, 100
    w = torch.rand(batch, m, j, k)
    a = torch.randn(batch, j, n)
    b = torch.randn(batch, k, n)
    set_tf32_enabled(False)
    gt = torch_lt2exp(w, a, b)
    set_tf32_enabled(allow_tf32)
    c = lt2exp(w, a, b, mode=mode)
    if allow_tf32:
        assert torch.allclose(gt, c, rtol=5e-4)
    else:
        assert torch.allclose(gt, c)

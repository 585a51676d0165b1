"""Global precision switch and reproducibility helper, mirroring triturus/utils.py:9-53.

`set_tf32_enabled(True)` selects the single-pass TF32 tensor-core path, `False` (the default, as in the
reference) the 3xTF32 split whose accuracy matches the reference's "ieee" dot.  The flag also flips torch's
own matmul / cuDNN TF32 switches, exactly as the reference does, so torch baselines run next to the
kernels at the matching precision.
"""

from __future__ import annotations

import os
import random

import numpy as np
import torch

_TRITURUS_TF32_ENABLED: bool = False


def ensure_reproducibility(
    *,
    seed: int = 42,
    determinism: bool = False,
    device: torch.device | int | str | None = None,
) -> None:
    """Seed python / numpy / torch and pick the default device (cuda when present), as
    triturus/utils.py:12-30 does."""
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if device is None:
        if torch.cuda.is_available():
            torch.set_default_device("cuda")
    else:
        torch.set_default_device(device)
    if determinism:
        torch.use_deterministic_algorithms(True, warn_only=True)
        torch.backends.cudnn.benchmark = False
        os.environ["CUBLAS_WORKSPACE_CONFIG"] = ":16:8"
    torch._dynamo.config.recompile_limit = 64


def set_tf32_enabled(allow_tf32: bool) -> None:
    """Module-global precision switch read by lm2exp / lt2exp (triturus/utils.py:33-44)."""
    global _TRITURUS_TF32_ENABLED
    allow = bool(allow_tf32)
    torch.set_float32_matmul_precision("high" if allow else "highest")
    torch.backends.cuda.matmul.allow_tf32 = allow
    torch.backends.cudnn.allow_tf32 = allow
    _TRITURUS_TF32_ENABLED = allow


def is_torch_tf32_enabled() -> bool:
    return bool(torch.backends.cuda.matmul.allow_tf32 and torch.backends.cudnn.allow_tf32)


def is_triturus_tf32_enabled() -> bool:
    return _TRITURUS_TF32_ENABLED


def resolve_precision(precision: str | None) -> int:
    """Map an explicit precision name, or the global flag when None, to the C-ABI precision code."""
    if precision is None:
        return 0 if _TRITURUS_TF32_ENABLED else 1
    if precision == "tf32":
        return 0
    if precision == "3xtf32":
        return 1
    raise ValueError(f"Unknown precision '{precision}' (expected 'tf32' or '3xtf32')")

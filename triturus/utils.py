"""`triturus.utils` names used by the reference's tests and benchmarks (triturus/utils.py:12-53)."""

from triturus_b200.utils import (
    ensure_reproducibility,
    is_torch_tf32_enabled,
    is_triturus_tf32_enabled,
    set_tf32_enabled,
)

__all__ = [
    "ensure_reproducibility",
    "is_torch_tf32_enabled",
    "is_triturus_tf32_enabled",
    "set_tf32_enabled",
]

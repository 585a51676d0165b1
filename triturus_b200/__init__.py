"""triturus_b200: the lm2exp / lt2exp log-space contractions of triturus as hand-written sm_100a CUDA.

Importing this package loads libtriturus_b200.so (built in-tree by `python -m triturus_b200.build`) and
registers `torch.ops.triturus.lm2exp` / `torch.ops.triturus.lt2exp`.  There is no fallback path.
"""

from . import lm2exp as _lm2exp_module
from . import lt2exp as _lt2exp_module
from ._native import NativeLibraryError, check_status, colmax
from .host import lm2exp_host, lt2exp_host
from .lm2exp import lm2exp
from .lt2exp import lt2exp
from .mm import mm
from .utils import (
    ensure_reproducibility,
    is_torch_tf32_enabled,
    is_triturus_tf32_enabled,
    set_tf32_enabled,
)

__all__ = [
    "NativeLibraryError",
    "check_status",
    "colmax",
    "ensure_reproducibility",
    "is_torch_tf32_enabled",
    "is_triturus_tf32_enabled",
    "lm2exp",
    "lm2exp_host",
    "lt2exp",
    "lt2exp_host",
    "mm",
    "set_tf32_enabled",
]

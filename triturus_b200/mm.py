"""mm host wrapper: same signature, checks and result as triturus/mm.py:181-214."""

from __future__ import annotations

import torch

from . import _native
from .utils import resolve_precision


def mm(a: torch.Tensor, b: torch.Tensor, *, precision: str | None = None) -> torch.Tensor:
    """out = a @ b for contiguous fp32 CUDA matrices a [M,K], b [K,N].

    The assertions are the reference's (triturus/mm.py:182-186).  The product runs through the lm2exp pipeline
    with the stabiliser, exp and log switched off.  With `set_tf32_enabled(True)` both operands are rounded to
    the nearest tf32 before a single tensor-core pass, which is what the reference's kernel does with cvt.rna
    (triturus/mm.py:152-154); otherwise the 3xTF32 split gives the accuracy of its "ieee" dot.  `precision`
    ("tf32" / "3xtf32") overrides the global flag."""
    assert len(a.shape) == len(b.shape) == 2
    assert a.shape[1] == b.shape[0]
    assert a.dtype == b.dtype == torch.float32
    assert a.device == b.device
    assert a.is_contiguous() and b.is_contiguous()
    _native._require_cuda(a, b)
    if a.numel() == 0 or b.numel() == 0:
        raise ValueError("mm: empty operands are not supported")
    return _native.mm_impl(a, b, resolve_precision(precision))

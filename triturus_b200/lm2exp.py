"""lm2exp host wrapper: same signature, checks and result as triturus/lm2exp.py:167-206."""

from __future__ import annotations

import torch

from . import _native
from .utils import resolve_precision


def lm2exp(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    precision: str | None = None,
    variant: int = 0,
    b_colmax: torch.Tensor | None = None,
    return_colmax: bool = False,
):
    """out[r,i,k] = log sum_j a[r,i,j] * exp(b[r,j,k]) for fp32 CUDA tensors a [R,I,J], b [R,J,K].

    The assertions are the reference's (triturus/lm2exp.py:168-172).  Inputs may have any strides and are
    never modified; the result is a new contiguous [R,I,K] tensor on the same device, produced
    asynchronously on torch's current stream.  `precision` overrides the global flag set by
    `triturus.utils.set_tf32_enabled` ("tf32" or "3xtf32"); `variant` pins the tile shape (0 = automatic).

    Chains of layers (no counterpart in the reference, whose kernel rescans every input for its column
    maxima, triturus/lm2exp.py:124-127): `return_colmax=True` returns `(out, m)` with `m[r,k] = max_i
    out[r,i,k]`, computed in the epilogue; passing that `m` as `b_colmax` to the call that uses `out` as its
    `b` skips that call's stabiliser pass.  `b_colmax` must hold the column maxima of `b` over its middle
    dimension (float32 [R,K]).
    """
    assert len(a.shape) == len(b.shape) == 3
    assert a.shape[0] == b.shape[0]
    assert a.shape[2] == b.shape[1]
    assert a.dtype == b.dtype == torch.float32
    assert a.device == b.device
    _native._require_cuda(a, b)
    prec = resolve_precision(precision)
    if a.numel() == 0 or b.numel() == 0:
        raise ValueError("lm2exp: empty operands are not supported")
    if b_colmax is None and not return_colmax:
        return _native.lm2exp_call(a, b, prec, int(variant))
    out, m = _native.lm2exp_chain_call(a, b, b_colmax, bool(return_colmax), prec, int(variant))
    return (out, m) if return_colmax else out

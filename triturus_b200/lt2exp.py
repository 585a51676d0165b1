"""lt2exp host wrapper: same signature, checks and result as triturus/lt2exp.py:519-630."""

from __future__ import annotations

import torch

from . import _native
from .utils import resolve_precision

_MODES = ("auto", "split", "unsplit")


def lt2exp(
    w: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    mode: str = "auto",
    precision: str | None = None,
    variant: int = 0,
    a_colmax: torch.Tensor | None = None,
    b_colmax: torch.Tensor | None = None,
    return_colmax: bool = False,
):
    """out[r,s,k] = log sum_{i,j} w[r,s,i,j] * exp(a[r,i,k]) * exp(b[r,j,k]) for fp32 CUDA tensors
    w [R,S,I,J], a [R,I,K], b [R,J,K].

    Assertions and the `mode` check are the reference's (triturus/lt2exp.py:522-541): an unknown mode
    raises ValueError.  The reference's "split" mode fills the GPU when R*S*K is small by cutting the
    contraction into NUM_SPLITS slices whose partial sums are merged in log space under a spin lock
    (triturus/lt2exp.py:498-506).  Here the slices share one stabiliser, add their partial sums into the
    result with fp32 reductions and a small second kernel takes the log.  mode="unsplit" never splits,
    mode="split" always does, mode="auto" splits when the output tiles would occupy fewer than half the SMs
    (and never under torch.use_deterministic_algorithms(True), because the order of the reductions is not
    fixed).  `variant` = SPLIT * 10000 + BN * 10 + MT pins the slice count and the tile shape explicitly.

    Chains of layers (no counterpart in the reference, whose kernels scan a and b for their column maxima in
    every call, triturus/lt2exp.py:305-311): `a_colmax` / `b_colmax` (float32 [R,K], both or neither) are the
    column maxima of `a` and `b` over their middle dimension, e.g. as returned by the calls that produced
    them, and replace the scan; `return_colmax=True` returns `(out, m)` with `m[r,k] = max_s out[r,s,k]`.
    """
    assert len(w.shape) == 4
    assert len(a.shape) == len(b.shape) == 3
    assert w.shape[0] == a.shape[0] == b.shape[0]
    assert w.shape[2] == a.shape[1]
    assert w.shape[3] == b.shape[1]
    assert a.shape[2] == b.shape[2]
    assert w.dtype == a.dtype == b.dtype == torch.float32
    assert w.device == a.device == b.device
    if mode not in _MODES:
        raise ValueError(f"Uknown mode '{mode}' for the l2exp kernel")
    # The reference flattens the last two dimensions of w with .view (triturus/lt2exp.py:549), which
    # raises when they are not jointly contiguous; keep that contract.
    w.view(w.shape[0], w.shape[1], -1)
    _native._require_cuda(w, a, b)
    prec = resolve_precision(precision)
    if w.numel() == 0 or a.numel() == 0 or b.numel() == 0:
        raise ValueError("lt2exp: empty operands are not supported")
    variant = int(variant)
    if variant < 10000:  # no explicit slice count: derive it from the mode
        if mode == "unsplit" or (mode == "auto" and torch.are_deterministic_algorithms_enabled()):
            variant += 10000
        elif mode == "split":
            variant += 9999 * 10000
    if a_colmax is None and b_colmax is None and not return_colmax:
        return _native.lt2exp_call(w, a, b, prec, variant)
    if (a_colmax is None) != (b_colmax is None):
        raise ValueError("lt2exp: a_colmax and b_colmax must be given together")
    out, m = _native.lt2exp_chain_call(w, a, b, a_colmax, b_colmax, bool(return_colmax), prec, variant)
    return (out, m) if return_colmax else out

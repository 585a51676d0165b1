"""CPU restatement of the reference's log-space contractions (TEST INFRASTRUCTURE, not a product path).

Two evaluators per op, both on CPU tensors:

* ``*_fp32``: the reference's own arithmetic, step for step, in float32 on torch CPU ops: column max ->
  clamp to +-1e38 -> exp of the shifted operand -> batched matmul -> log -> add the max back.
  lm2exp follows baselines/lm2exp.py:11-14; lt2exp follows baselines/lt2exp.py:15-25 (which materialises
  the [R, I*J, K] Khatri-Rao operand before one bmm).  This is the reference's CPU path and the timed
  CPU baseline.
* ``*_fp64``: the same formula in float64 with the clamp widened to +-1e300 (no fp32 range to protect),
  evaluated in batch chunks so the lt2exp intermediate stays small.  This is the accuracy yardstick for
  the tolerances (abs <= 2e-3 for TF32, <= 1e-4 for 3xTF32, in log space).

Pinning: the reference holds no golden vectors for this path; its tests compare against these torch
baselines on seeded inputs (tests/lm2exp.py:13-23, tests/lt2exp.py:19-40).  The fixtures under
tests/golden/ were produced by importing the reference's baselines themselves (tests/golden/make_golden.py)
and tests/test_oracle_golden.py checks every function here against them.
"""

from __future__ import annotations

import torch

FP32_CLAMP = 1e38  # baselines/lm2exp.py:12, baselines/lt2exp.py:16,19
FP64_CLAMP = 1e300


def _stabiliser(x: torch.Tensor, bound: float) -> torch.Tensor:
    """Clamped maximum over dim 1 with the dim kept, i.e. one value per (batch, column)."""
    return x.amax(dim=1, keepdim=True).clamp(min=-bound, max=bound)


def lm2exp_fp32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """baselines/lm2exp.py:4-14 in float32: a [R,I,J], b [R,J,K] -> [R,I,K]."""
    _check_lm(a, b)
    m = _stabiliser(b, FP32_CLAMP)
    lin = torch.bmm(a, (b - m).exp())
    return lin.log() + m


def lm2exp_fp64(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Float64 evaluation of the lm2exp formula (README.md:12); returns float64."""
    _check_lm(a, b)
    a64, b64 = a.double(), b.double()
    m = _stabiliser(b64, FP64_CLAMP)
    return torch.bmm(a64, (b64 - m).exp()).log() + m


def lt2exp_fp32(w: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """baselines/lt2exp.py:4-25 in float32: w [R,S,I,J], a [R,I,K], b [R,J,K] -> [R,S,K].

    Like the reference it forms the full outer product of the two exp'd operands, [R, I*J, K], and
    contracts it with w flattened to [R, S, I*J] in a single bmm.
    """
    _check_lt(w, a, b)
    R, S, I, J = w.shape
    K = a.shape[2]
    ma = _stabiliser(a, FP32_CLAMP)
    mb = _stabiliser(b, FP32_CLAMP)
    ea = (a - ma).exp()
    eb = (b - mb).exp()
    kr = (ea[:, :, None, :] * eb[:, None, :, :]).reshape(R, I * J, K)
    lin = torch.bmm(w.reshape(R, S, I * J), kr)
    return ma + mb + lin.log()


def lt2exp_fp64(w: torch.Tensor, a: torch.Tensor, b: torch.Tensor, *, chunk: int = 1) -> torch.Tensor:
    """Float64 evaluation of the lt2exp formula (README.md:13), `chunk` batch entries at a time."""
    _check_lt(w, a, b)
    R, S, I, J = w.shape
    K = a.shape[2]
    out = torch.empty((R, S, K), dtype=torch.float64)
    for r0 in range(0, R, chunk):
        sl = slice(r0, min(R, r0 + chunk))
        a64, b64, w64 = a[sl].double(), b[sl].double(), w[sl].double()
        ma = _stabiliser(a64, FP64_CLAMP)
        mb = _stabiliser(b64, FP64_CLAMP)
        ea = (a64 - ma).exp()
        eb = (b64 - mb).exp()
        # contract j first, then i: [r,S,I,J] x [r,J,K] -> [r,S,I,K]; weight by ea and sum over i
        t = torch.einsum("rsij,rjk->rsik", w64, eb)
        lin = (t * ea[:, None, :, :]).sum(dim=2)
        out[sl] = ma + mb + lin.log()
    return out


def _check_lm(a: torch.Tensor, b: torch.Tensor) -> None:
    if a.dim() != 3 or b.dim() != 3 or a.shape[0] != b.shape[0] or a.shape[2] != b.shape[1]:
        raise ValueError(f"lm2exp: incompatible shapes {tuple(a.shape)} and {tuple(b.shape)}")
    if a.dtype != torch.float32 or b.dtype != torch.float32:
        raise ValueError("lm2exp: operands must be float32")


def _check_lt(w: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> None:
    ok = (
        w.dim() == 4
        and a.dim() == 3
        and b.dim() == 3
        and w.shape[0] == a.shape[0] == b.shape[0]
        and w.shape[2] == a.shape[1]
        and w.shape[3] == b.shape[1]
        and a.shape[2] == b.shape[2]
    )
    if not ok:
        raise ValueError(f"lt2exp: incompatible shapes {tuple(w.shape)}, {tuple(a.shape)}, {tuple(b.shape)}")
    if not (w.dtype == a.dtype == b.dtype == torch.float32):
        raise ValueError("lt2exp: operands must be float32")


def compare_logspace(got: torch.Tensor, want: torch.Tensor, atol: float) -> dict:
    """Compare a result with a reference in log space.

    Passes when there is no NaN in `got`, the -inf (and +inf) positions are identical, and every finite
    entry is within `atol` in absolute terms.  Returns a dict with `ok`, `max_abs_err`, `nan`, and
    `inf_mismatch` so tests can print what failed.
    """
    got64 = got.detach().cpu().double()
    want64 = want.detach().cpu().double()
    if got64.shape != want64.shape:
        return {"ok": False, "reason": f"shape {tuple(got64.shape)} != {tuple(want64.shape)}"}
    nan = int(torch.isnan(got64).sum())
    inf_mismatch = int(((got64 == float("-inf")) != (want64 == float("-inf"))).sum())
    inf_mismatch += int(((got64 == float("inf")) != (want64 == float("inf"))).sum())
    finite = torch.isfinite(want64) & torch.isfinite(got64)
    err = (got64[finite] - want64[finite]).abs()
    max_err = float(err.max()) if err.numel() else 0.0
    ok = nan == 0 and inf_mismatch == 0 and max_err <= atol
    return {"ok": ok, "max_abs_err": max_err, "nan": nan, "inf_mismatch": inf_mismatch, "atol": atol}

"""GPU regression over the reference's benchmark sweeps (benchmarks/lm2exp.py:26-56, benchmarks/lt2exp.py:32-63):
every shape of the four families is run through the drop-in entry points, both TF32 settings, and compared with
the float64 oracle (whole result for small shapes, a batch and row subset for the large ones).

Tolerance: the stated absolute tolerances in log space against the float64 evaluation, 1e-4 for 3xTF32 and 2e-3
for plain TF32, as written, whatever the length of the contraction.  (The tensor core's fp32 accumulator truncates
instead of rounding, which over L terms loses ~1.2e-8 * L relatively; contractions of more than 32 K terms
therefore run on the kernels that re-sum their accumulator in chunks with rounded adds, in both precisions.)"""

import pytest
import torch

from conftest import ATOL
from oracle import logspace_oracle as orc
from triturus_b200.sweeps import lm2exp_sweep, lt2exp_sweep

pytestmark = pytest.mark.gpu


def _ids(pts):
    return [f"{p.family.replace(' ', '').replace(',', '_')}-{'x'.join(str(v) for v in p.dims.values())}" for p in pts]


LM = lm2exp_sweep()
LT = lt2exp_sweep()


def _tol(allow_tf32):
    return ATOL["tf32"] if allow_tf32 else ATOL["3xtf32"]


@pytest.mark.parametrize("allow_tf32", [False, True])
@pytest.mark.parametrize("pt", LM, ids=_ids(LM))
def test_lm2exp_sweep_shape(pt, allow_tf32):
    from triturus.lm2exp import lm2exp
    from triturus.utils import set_tf32_enabled
    import triturus_b200 as tb

    a, b = pt.make_inputs("cpu")
    set_tf32_enabled(allow_tf32)
    out = lm2exp(a.cuda(), b.cuda())
    set_tf32_enabled(False)
    tb.check_status()
    assert out.shape == (pt.dims["batch"], pt.dims["m"], pt.dims["n"])
    # float64 oracle on at most 4 batch entries and 256 rows (the columns are all checked)
    rs = sorted({0, pt.dims["batch"] // 2, pt.dims["batch"] - 1})
    rows = slice(0, min(pt.dims["m"], 256))
    want = orc.lm2exp_fp64(a[rs][:, rows].contiguous(), b[rs])
    res = orc.compare_logspace(out[rs][:, rows].cpu(), want, _tol(allow_tf32))
    assert res["ok"], res
    assert not torch.isnan(out).any()


@pytest.mark.parametrize("allow_tf32", [False, True])
@pytest.mark.parametrize("pt", LT, ids=_ids(LT))
def test_lt2exp_sweep_shape(pt, allow_tf32):
    from triturus.lt2exp import lt2exp
    from triturus.utils import set_tf32_enabled
    import triturus_b200 as tb

    w, a, b = pt.make_inputs("cpu")
    set_tf32_enabled(allow_tf32)
    out = lt2exp(w.cuda(), a.cuda(), b.cuda())
    set_tf32_enabled(False)
    tb.check_status()
    assert out.shape == (pt.dims["batch"], pt.dims["m"], pt.dims["n"])
    big = pt.dims["j"] * pt.dims["k"] * pt.dims["m"] * pt.dims["n"] > (1 << 28)
    rs = [0] if big else sorted({0, pt.dims["batch"] - 1})
    rows = slice(0, min(pt.dims["m"], 64 if big else 256))
    want = orc.lt2exp_fp64(w[rs][:, rows].contiguous(), a[rs], b[rs])
    res = orc.compare_logspace(out[rs][:, rows].cpu(), want, _tol(allow_tf32))
    assert res["ok"], res
    assert not torch.isnan(out).any()

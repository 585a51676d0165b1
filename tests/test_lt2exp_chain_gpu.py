"""GPU tests of lt2exp used as a link of a chain of layers: caller-supplied column maxima of a and b
(`a_colmax`, `b_colmax`) and the column maxima of the result from the epilogue (`return_colmax`), for the
shared-memory kernels, the TMEM-operand kernels and the split contraction.  Tolerances as everywhere: abs
2e-3 (TF32) / 1e-4 (3xTF32) in log space against float64, -inf positions identical, no NaN."""

import pytest
import torch

from conftest import ATOL
from oracle import logspace_oracle as orc

pytestmark = pytest.mark.gpu


def _inputs(R, S, I, J, K, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.rand(R, S, I, J, generator=g) + 0.01
    a = torch.randn(R, I, K, generator=g) * 4.0 - 20.0 * torch.rand(R, 1, K, generator=g)
    b = torch.randn(R, J, K, generator=g) * 4.0 + 30.0 * torch.randn(R, 1, K, generator=g)
    a[0, :, 3] = float("-inf")  # a dead column: the result column is -inf and so is its maximum
    return w, a, b


# (shape, variant, precisions): shared-memory tiles, TMEM-operand tiles (TF32 only), split contraction
CASES = [
    ((2, 100, 20, 24, 200), 0, ("tf32", "3xtf32")),
    ((2, 300, 16, 40, 300), 11281, ("tf32", "3xtf32")),
    ((2, 300, 16, 40, 300), 11282, ("tf32", "3xtf32")),
    ((2, 140, 16, 40, 300), 12561, ("tf32", "3xtf32")),
    ((1, 300, 16, 40, 520), 12562, ("tf32",)),
    ((2, 130, 16, 40, 300), 11283, ("tf32",)),
    ((2, 300, 16, 40, 300), 11284, ("tf32",)),
    ((2, 130, 16, 40, 300), 11285, ("tf32",)),
    ((1, 64, 64, 64, 128), 9999 * 10000, ("tf32", "3xtf32")),   # split contraction (three launches + fill)
    ((1, 200, 32, 64, 130), 4 * 10000 + 1283, ("tf32",)),        # split, TMEM-operand kernel
]
PARAMS = [(shape, variant, prec) for shape, variant, precs in CASES for prec in precs]


@pytest.mark.parametrize("shape,variant,precision", PARAMS)
def test_returned_colmax_and_supplied_maxima(shape, variant, precision):
    import triturus_b200 as tb

    w, a, b = _inputs(*shape, seed=sum(shape))
    wd, ad, bd = w.cuda(), a.cuda(), b.cuda()
    want = orc.lt2exp_fp64(w, a, b)

    plain = tb.lt2exp(wd, ad, bd, precision=precision, variant=variant)
    out, m = tb.lt2exp(wd, ad, bd, precision=precision, variant=variant, return_colmax=True)
    tb.check_status()
    res = orc.compare_logspace(out.cpu(), want, ATOL[precision])
    assert res["ok"], res
    assert torch.equal(m, out.amax(dim=1))              # the maximum of the stored values, bit for bit
    assert torch.all(m[0, 3] == float("-inf"))
    if variant // 10000 <= 1:                           # unsplit results are deterministic
        assert torch.equal(out, plain)

    got = tb.lt2exp(wd, ad, bd, precision=precision, variant=variant,
                    a_colmax=ad.amax(dim=1), b_colmax=bd.amax(dim=1))
    tb.check_status()
    res = orc.compare_logspace(got.cpu(), want, ATOL[precision])
    assert res["ok"], res
    if variant // 10000 <= 1:
        assert torch.equal(got, plain)                  # same stabilisers, same kernel, same bits


@pytest.mark.parametrize("precision", ["tf32", "3xtf32"])
def test_mixed_chain_lt2exp_into_lm2exp(precision):
    """A Tucker layer feeding a dense layer: the maxima of the lt2exp result are the stabiliser of the lm2exp."""
    import triturus_b200 as tb

    w, a, b = _inputs(3, 260, 24, 24, 700, seed=9)
    g = torch.Generator().manual_seed(10)
    dense = torch.softmax(torch.randn(3, 384, 260, generator=g), dim=-1)
    x1, m1 = tb.lt2exp(w.cuda(), a.cuda(), b.cuda(), precision=precision, return_colmax=True)
    x2, m2 = tb.lm2exp(dense.cuda(), x1, precision=precision, b_colmax=m1, return_colmax=True)
    x2_plain = tb.lm2exp(dense.cuda(), x1, precision=precision)
    tb.check_status()
    assert torch.equal(m2, x2.amax(dim=1))
    x1_64 = orc.lt2exp_fp64(w, a, b)
    m64 = x1_64.amax(dim=1, keepdim=True).clamp(min=-1e300, max=1e300)
    x2_64 = torch.bmm(dense.double(), (x1_64 - m64).exp()).log() + m64
    res = orc.compare_logspace(x2.cpu(), x2_64, 2 * ATOL[precision])
    assert res["ok"], res
    res = orc.compare_logspace(x2.cpu(), x2_plain.cpu().double(), 2 * ATOL[precision])
    assert res["ok"], res

    # and back into a Tucker layer: both of its operands come with their maxima
    w2 = torch.rand(3, 100, 24, 24, generator=g)
    y, my = tb.lt2exp(w2.cuda(), x2[:, :24].contiguous(), x2[:, 24:48].contiguous(), precision=precision,
                      a_colmax=x2[:, :24].amax(dim=1), b_colmax=x2[:, 24:48].amax(dim=1), return_colmax=True)
    y_plain = tb.lt2exp(w2.cuda(), x2[:, :24].contiguous(), x2[:, 24:48].contiguous(), precision=precision)
    tb.check_status()
    assert torch.equal(y, y_plain) and torch.equal(my, y.amax(dim=1))


def test_argument_checks():
    import triturus_b200 as tb

    w, a, b = _inputs(1, 16, 8, 8, 32, seed=1)
    with pytest.raises(ValueError):
        tb.lt2exp(w.cuda(), a.cuda(), b.cuda(), a_colmax=a.cuda().amax(dim=1))
    with pytest.raises(ValueError):
        tb.lt2exp(w.cuda(), a.cuda(), b.cuda(), a_colmax=torch.zeros(1, 31, device="cuda"),
                  b_colmax=torch.zeros(1, 31, device="cuda"))

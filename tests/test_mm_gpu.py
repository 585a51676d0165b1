"""GPU: the plain matrix product that falls out of the contraction pipeline (the reference's triturus/mm.py),
against float64 and with the reference's own acceptance test (tests/mm.py:8-16)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("allow_tf32", [False, True])
def test_mm_reference_shape_and_bound(allow_tf32):
    """The reference's test: 150 x 100 x 200, operands from U(0, 1), against torch.mm at the matching TF32 setting.
    With the flag off the bound is the reference's (torch.allclose defaults, rtol 1e-5).  With the flag on, two
    single-pass TF32 products (cuBLAS and this kernel) are compared: they agree to a few 1e-6 relative, not always
    inside 1e-5, so the bound there is the rtol 5e-4 the reference uses for its TF32 paths (tests/lm2exp.py:21),
    plus a check that this kernel is as close to the float64 product as cuBLAS is."""
    from triturus.mm import mm
    from triturus.utils import set_tf32_enabled
    import triturus_b200 as tb

    set_tf32_enabled(allow_tf32)
    g = torch.Generator().manual_seed(42)
    a = torch.rand(150, 100, generator=g).cuda()
    b = torch.rand(100, 200, generator=g).cuda()
    gt = torch.mm(a, b)
    c = mm(a, b)
    set_tf32_enabled(False)
    tb.check_status()
    assert c.shape == (150, 200) and c.is_contiguous()
    if not allow_tf32:
        assert torch.allclose(gt, c)
    else:
        assert torch.allclose(gt, c, rtol=5e-4)
        want = a.double() @ b.double()
        assert (c.double() - want).abs().max() <= 1.5 * (gt.double() - want).abs().max() + 1e-6


@pytest.mark.parametrize("precision,rtol", [("tf32", 2e-3), ("3xtf32", 2e-5)])
@pytest.mark.parametrize("shape", [(1, 1, 1), (3, 5, 7), (257, 33, 130), (300, 1000, 515), (1024, 2048, 512)])
def test_mm_against_float64(shape, precision, rtol):
    """Signed operands, ragged sizes, results compared with the float64 product relative to the size of the terms."""
    import triturus_b200 as tb

    M, K, N = shape
    g = torch.Generator().manual_seed(M + K + N)
    a = torch.randn(M, K, generator=g)
    b = torch.randn(K, N, generator=g)
    got = tb.mm(a.cuda(), b.cuda(), precision=precision).cpu().double()
    tb.check_status()
    want = a.double() @ b.double()
    scale = (a.double().abs() @ b.double().abs())  # sum of |terms|: the natural yardstick for a signed sum
    assert ((got - want).abs() <= rtol * scale + 1e-30).all()


def test_mm_keeps_the_reference_assertions():
    import triturus_b200 as tb

    a = torch.rand(4, 6).cuda()
    with pytest.raises(AssertionError):
        tb.mm(a, torch.rand(5, 3).cuda())          # inner dimensions differ
    with pytest.raises(AssertionError):
        tb.mm(a, torch.rand(3, 6).cuda().t())      # not contiguous (triturus/mm.py:186)
    with pytest.raises(AssertionError):
        tb.mm(a.double(), torch.rand(6, 3).cuda().double())

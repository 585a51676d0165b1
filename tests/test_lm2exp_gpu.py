"""GPU parity tests for lm2exp: the CUDA path (through the C ABI) against the golden fixtures produced by
the reference's baseline, against the float64 oracle, and through size-independent properties at the full
benchmark sizes.  Tolerances (absolute, log space, vs float64): 2e-3 for TF32, 1e-4 for 3xTF32; -inf
positions must match exactly and no NaN may appear."""

import pytest
import torch

from conftest import ATOL, LM_GOLDEN, load_golden
from oracle import logspace_oracle as orc

pytestmark = pytest.mark.gpu

PRECISIONS = ["tf32", "3xtf32"]
VARIANTS = [0, 1281, 1282, 2561, 2562, 2564, 101282, 202561]


def _run(a, b, **kw):
    import triturus_b200 as tb

    out = tb.lm2exp(a.cuda(), b.cuda(), **kw)
    tb.check_status()
    return out.cpu()


def _assert_close(got, a, b, precision, want64=None):
    want64 = orc.lm2exp_fp64(a, b) if want64 is None else want64
    res = orc.compare_logspace(got, want64, ATOL[precision])
    assert res["ok"], res


@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("name", LM_GOLDEN)
def test_golden(name, precision):
    g = load_golden(name)
    got = _run(g["a"], g["b"], precision=precision)
    # against the reference baseline's stored output (fp32, itself ~1e-5 from exact)
    res = orc.compare_logspace(got, g["out"], ATOL[precision] + 2e-5)
    assert res["ok"], res
    _assert_close(got, g["a"], g["b"], precision)


@pytest.mark.parametrize("shape", [(1, 256, 32, 256), (2, 300, 100, 260), (3, 257, 33, 516), (2, 1000, 250, 1000),
                                   (1, 130, 1024, 40), (5, 300, 171, 530)])
def test_tmem_operand_pair_kernel(shape):
    """Variant 2566: the CTA-pair kernel that keeps exp(b - m) in tensor memory (plain TF32), on ragged shapes with
    isolated -inf entries, an all -inf column, rows past I, columns past K and a partial last k-block.  Its
    arithmetic is that of the shared-memory pair kernel (2564) in the same order, so the two agree bit for bit."""
    import triturus_b200 as tb

    R, I, J, K = shape
    g = torch.Generator().manual_seed(sum(shape))
    a = torch.rand(R, I, J, generator=g)
    b = torch.randn(R, J, K, generator=g) * 6.0 + 50.0 * torch.randn(R, 1, K, generator=g)
    b[0, :, min(3, K - 1)] = float("-inf")
    b[torch.rand(R, J, K, generator=g) < 0.01] = float("-inf")
    from triturus_b200 import _native

    assert _native.LIB.triturus_b200_lm2exp_plan(R, I, J, K, 0, 2566) == 102566
    got = tb.lm2exp(a.cuda(), b.cuda(), precision="tf32", variant=2566)
    same = tb.lm2exp(a.cuda(), b.cuda(), precision="tf32", variant=2564)
    tb.check_status()
    assert torch.all(got[0, :, min(3, K - 1)] == float("-inf"))
    _assert_close(got.cpu(), a, b, "tf32")
    assert torch.equal(got, same)
    with pytest.raises(tb.NativeLibraryError):
        tb.lm2exp(a.cuda(), b.cuda(), precision="3xtf32", variant=2566)


def _optimistic_cases():
    """(name, a, b, takes_the_exact_passes) for the optimistic stabiliser: columns whose later rows stay below,
    exceed moderately, or overflow past the maximum of their first 32 rows."""
    g = torch.Generator().manual_seed(2567)
    rnd = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    uni = lambda *s: torch.rand(*s, generator=g)  # noqa: E731
    b = rnd(3, 250, 520) * 6.0 + 50.0 * rnd(3, 1, 520)
    b[0, :, 3] = float("-inf")
    b[uni(3, 250, 520) < 0.01] = float("-inf")
    yield "random", uni(3, 300, 250), b, False
    b = rnd(2, 256, 512)
    b[:, 100:] += 30.0
    yield "later-rows-30-above", uni(2, 512, 256), b, False
    b = rnd(2, 256, 512)
    b[:, 64:] += 70.0
    yield "later-rows-70-above", uni(2, 512, 256) * 1e-3, b, False
    b = torch.arange(1024, dtype=torch.float32).view(1, 1024, 1).expand(2, 1024, 512).contiguous() + rnd(2, 1024, 512)
    yield "ramp-of-1000", uni(2, 512, 1024), b, True
    b = rnd(2, 256, 512)
    b[:, :32] = float("-inf")
    yield "first-rows-all-neg-inf", uni(2, 512, 256), b, True
    b = rnd(1, 256, 512)
    b[0, 200, 77] = 500.0
    yield "one-spike", uni(1, 512, 256), b, True
    b = rnd(2, 40, 300)
    yield "short-contraction", uni(2, 512, 40), b, False
    b = rnd(40, 8, 512)
    b[:, 5] += 200.0
    yield "one-k-block-per-tile", uni(40, 512, 8), b, False


@pytest.mark.parametrize("case", list(_optimistic_cases()), ids=lambda c: c[0])
def test_optimistic_stabiliser(case):
    """Variant 2567: no pre-pass; the stabiliser of a column is the maximum of its first 32 rows, and a result that
    overflowed makes the conditional launch behind it (the same kernel with an exact max pass inside) redo the call.
    Either way the result is within the TF32 tolerance of float64; where the exact pass ran it is bit for bit the
    result of the pre-pass variant (the maxima are the same numbers)."""
    import triturus_b200 as tb
    from triturus_b200 import _native

    name, a, b, exact = case
    R, I, J = a.shape
    K = b.shape[2]
    assert _native.LIB.triturus_b200_lm2exp_plan(R, I, J, K, 0, 2567) == 2567
    assert _native.LIB.triturus_b200_lm2exp_plan(R, I, J, K, 0, 102567) == 102566
    assert _native.LIB.triturus_b200_lm2exp_launches(R, I, J, K, 0, 2567) == 2
    ad, bd = a.cuda(), b.cuda()
    got = tb.lm2exp(ad, bd, precision="tf32", variant=2567)
    tb.check_status()
    _assert_close(got.cpu(), a, b, "tf32")
    pre = tb.lm2exp(ad, bd, precision="tf32", variant=102566)
    tb.check_status()
    assert torch.equal(torch.isinf(got), torch.isinf(pre))
    if exact:
        assert torch.equal(got, pre)
    elif name in ("random", "later-rows-30-above", "later-rows-70-above"):
        # the optimistic result was kept (another stabiliser, so other roundings): the exact passes did not run
        assert not torch.equal(got, pre)
    # a clean call afterwards starts from a cleared flag
    b2 = torch.randn(R, J, K, generator=torch.Generator().manual_seed(1))
    got2 = tb.lm2exp(ad, b2.cuda(), precision="tf32", variant=2567)
    tb.check_status()
    _assert_close(got2.cpu(), a, b2, "tf32")
    with pytest.raises(tb.NativeLibraryError):
        tb.lm2exp(ad, bd, precision="3xtf32", variant=2567)


@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("case", list(_optimistic_cases()), ids=lambda c: c[0])
def test_optimistic_prepass_of_the_shared_memory_pair_kernel(case, precision):
    """Stabiliser code 4 (variant 402564; automatic for 3xTF32 on pair tiles): the pre-pass takes the column maxima
    over the first 32 rows of b only, the pair kernel checks its results for overflow, and the full pre-pass and
    the contraction with its maxima follow as conditional launches.  Where they ran, the result is bit for bit
    that of the pre-pass variant 102564."""
    import triturus_b200 as tb
    from triturus_b200 import _native

    name, a, b, exact = case
    R, I, J = a.shape
    K = b.shape[2]
    prec = 0 if precision == "tf32" else 1
    if J < 128:
        assert _native.LIB.triturus_b200_lm2exp_plan(R, I, J, K, prec, 402564) == 102564  # nothing to save
        return
    assert _native.LIB.triturus_b200_lm2exp_plan(R, I, J, K, prec, 402564) == 402564
    assert _native.LIB.triturus_b200_lm2exp_launches(R, I, J, K, prec, 402564) == 4
    ad, bd = a.cuda(), b.cuda()
    got = tb.lm2exp(ad, bd, precision=precision, variant=402564)
    tb.check_status()
    _assert_close(got.cpu(), a, b, precision)
    pre = tb.lm2exp(ad, bd, precision=precision, variant=102564)
    tb.check_status()
    assert torch.equal(torch.isinf(got), torch.isinf(pre))
    if exact:
        assert torch.equal(got, pre)
    elif name in ("random", "later-rows-30-above", "later-rows-70-above"):
        assert not torch.equal(got, pre)  # the optimistic result was kept
    b2 = torch.randn(R, J, K, generator=torch.Generator().manual_seed(1))
    got2 = tb.lm2exp(ad, b2.cuda(), precision=precision, variant=402564)
    tb.check_status()
    _assert_close(got2.cpu(), a, b2, precision)


def test_optimistic_stabiliser_is_the_automatic_choice_for_tf32_pairs():
    """cfg2's shape: plain TF32 runs the optimistic TMEM-operand kernel, 3xTF32 the shared-memory pair kernel with
    the pre-pass; a supplied stabiliser or a forced pre-pass leaves the optimistic form out."""
    from triturus_b200 import _native

    L = _native.LIB
    assert L.triturus_b200_lm2exp_plan(32, 1024, 1024, 1024, 0, 0) == 2567
    assert L.triturus_b200_lm2exp_plan(32, 1024, 1024, 1024, 1, 0) == 402564  # 3xTF32: optimistic 32-row pre-pass
    assert L.triturus_b200_lm2exp_plan(32, 1024, 1024, 1024, 1, 2564) == 102564  # an explicit tile keeps the full one
    assert L.triturus_b200_lm2exp_launches(32, 1024, 1024, 1024, 1, 0) == 4
    assert L.triturus_b200_lm2exp_plan(32, 1024, 1024, 1024, 0, 100000) == 102566
    assert L.triturus_b200_lm2exp_launches(32, 1024, 1024, 1024, 0, 0) == 2
    assert L.triturus_b200_lm2exp_chain_launches(32, 1024, 1024, 1024, 0, 0, 1, 0) == 1


def _optimistic_fused_cases():
    g = torch.Generator().manual_seed(3000)
    rnd = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    uni = lambda *s: torch.rand(*s, generator=g)  # noqa: E731
    b = rnd(3, 250, 700) * 6.0 + 50.0 * rnd(3, 1, 700)
    b[0, :, 3] = float("-inf")
    b[uni(3, 250, 700) < 0.01] = float("-inf")
    yield "random", uni(3, 200, 250), b, False
    b = torch.arange(512, dtype=torch.float32).view(1, 512, 1).expand(2, 512, 300).contiguous() + rnd(2, 512, 300)
    yield "ramp-of-500", uni(2, 100, 512), b, True
    b = rnd(2, 256, 300)
    b[:, :32] = float("-inf")
    yield "first-rows-all-neg-inf", uni(2, 256, 256), b, True
    b = rnd(2, 256, 300)
    b[:, 64:] += 60.0
    yield "later-rows-60-above", uni(2, 256, 256) * 1e-3, b, False


@pytest.mark.parametrize("tile", [0, 1281, 1282, 2561])
@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("case", list(_optimistic_fused_cases()), ids=lambda c: c[0])
def test_optimistic_fused_max_pass(case, precision, tile):
    """Stabiliser code 3: the fused max pass of the single-CTA kernel scans the first k-block of a slab only; a
    result that overflowed makes the conditional launch behind it redo the call with the full pass (code 2), whose
    result it then equals bit for bit."""
    import triturus_b200 as tb
    from triturus_b200 import _native

    name, a, b, exact = case
    if precision == "3xtf32" and tile == 2561:
        pytest.skip("3xTF32 tiles have 128 columns")
    R, I, J = a.shape
    K = b.shape[2]
    prec = 0 if precision == "tf32" else 1
    assert _native.LIB.triturus_b200_lm2exp_plan(R, I, J, K, prec, 300000 + tile) // 100000 == 3
    assert _native.LIB.triturus_b200_lm2exp_launches(R, I, J, K, prec, 300000 + tile) == 2
    ad, bd = a.cuda(), b.cuda()
    got = tb.lm2exp(ad, bd, precision=precision, variant=300000 + tile)
    tb.check_status()
    _assert_close(got.cpu(), a, b, precision)
    full = tb.lm2exp(ad, bd, precision=precision, variant=200000 + tile)
    tb.check_status()
    assert torch.equal(torch.isinf(got), torch.isinf(full))
    if exact:
        assert torch.equal(got, full)
    else:
        assert not torch.equal(got, full)  # the optimistic result was kept
    # the next call starts from a flag that is down
    b2 = torch.randn(R, J, K, generator=torch.Generator().manual_seed(2))
    got2 = tb.lm2exp(ad, b2.cuda(), precision=precision, variant=300000 + tile)
    tb.check_status()
    _assert_close(got2.cpu(), a, b2, precision)


def test_optimistic_fused_max_pass_is_automatic_for_long_tf32_launches():
    """One 128-row block, long launch: plain TF32 takes the optimistic max pass, 3xTF32 and short or small problems
    the full one.  From two row blocks on (cfg3) the pair kernels with their optimistic stabilisers take over."""
    from triturus_b200 import _native

    L = _native.LIB
    assert L.triturus_b200_lm2exp_plan(256, 128, 256, 8192, 0, 0) // 100000 == 3
    assert L.triturus_b200_lm2exp_plan(256, 128, 256, 8192, 1, 0) // 100000 == 2
    assert L.triturus_b200_lm2exp_launches(256, 128, 256, 8192, 0, 0) == 2
    assert L.triturus_b200_lm2exp_plan(4, 256, 256, 256, 0, 0) == 201281  # cfg1: less than one wave
    assert L.triturus_b200_lm2exp_plan(256, 128, 64, 8192, 0, 0) // 100000 == 2  # two k-blocks: nothing to save
    assert L.triturus_b200_lm2exp_plan(128, 256, 256, 8192, 0, 0) == 2567  # cfg3
    assert L.triturus_b200_lm2exp_plan(128, 256, 256, 8192, 1, 0) == 402564
    assert L.triturus_b200_lm2exp_plan(128, 256, 256, 8192, 0, 100000) % 10 == 2  # forced pre-pass: a single-CTA tile as before
    assert L.triturus_b200_lm2exp_plan(128, 256, 256, 8192, 0, 200000) == 201282
    assert L.triturus_b200_lm2exp_chain_launches(128, 256, 256, 8192, 0, 300000, 1, 0) < 0  # stabiliser supplied


def test_tmem_operand_pair_kernel_unaligned_result():
    """K not a multiple of 4: the wrapper pads b, the result rows are not 16-byte aligned and are written row by row."""
    g = torch.Generator().manual_seed(99)
    a = torch.rand(2, 270, 70, generator=g)
    b = torch.randn(2, 70, 263, generator=g) * 4.0
    got = _run(a, b, precision="tf32", variant=2566)
    _assert_close(got, a, b, "tf32")


@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("shape", [(40, 300, 100, 520), (64, 512, 75, 256), (33, 260, 1030, 130)])
def test_pair_kernel_on_batches_of_several_waves(shape, precision):
    """The CTA-pair kernel on batches of several waves of tiles (the pre-pass and the contraction kernel launched
    as programmatic dependents): ragged J and K, late entries with all -inf columns, huge column offsets.  The
    pre-pass maxima are exact, so the result is bit for bit that of a call that is given the column maxima."""
    import triturus_b200 as tb

    R, I, J, K = shape
    g = torch.Generator().manual_seed(sum(shape))
    a = torch.rand(R, I, J, generator=g)
    b = torch.randn(R, J, K, generator=g) * 8.0 + 150.0 * torch.randn(R, 1, K, generator=g)
    b[R - 1, :, 5] = float("-inf")
    b[R // 2, :, K - 1] = float("-inf")
    b[torch.rand(R, J, K, generator=g) < 0.02] = float("-inf")
    ad, bd = a.cuda(), b.cuda()
    got = tb.lm2exp(ad, bd, precision=precision, variant=2564)
    tb.check_status()
    assert torch.all(got[R - 1, :, 5] == float("-inf")) and torch.all(got[R // 2, :, K - 1] == float("-inf"))
    rs = [0, R // 2, R - 1]
    res = orc.compare_logspace(got[rs].cpu(), orc.lm2exp_fp64(a[rs], b[rs]), ATOL[precision])
    assert res["ok"], res
    same = tb.lm2exp(ad, bd, precision=precision, variant=2564, b_colmax=bd.amax(dim=1))
    tb.check_status()
    assert torch.equal(got, same)


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("precision", PRECISIONS)
def test_variants_on_ragged_shape(precision, variant):
    g = torch.Generator().manual_seed(7)
    a = torch.rand(5, 300, 171, generator=g)
    b = torch.randn(5, 171, 530, generator=g) * 5.0 + 100.0 * torch.randn(5, 1, 530, generator=g)
    got = _run(a, b, precision=precision, variant=variant)
    _assert_close(got, a, b, precision)


@pytest.mark.parametrize("shape", [(1, 1, 1, 1), (1, 1, 33, 5), (2, 129, 31, 3), (3, 7, 64, 257), (1, 260, 5, 1030),
                                   (2, 128, 32, 128), (4, 256, 96, 256)])
@pytest.mark.parametrize("precision", PRECISIONS)
def test_edge_shapes(shape, precision):
    R, I, J, K = shape
    g = torch.Generator().manual_seed(R * 1000 + I + J + K)
    a = torch.rand(R, I, J, generator=g) + 0.01
    b = torch.randn(R, J, K, generator=g) * 3.0
    got = _run(a, b, precision=precision)
    assert got.shape == (R, I, K) and got.is_contiguous()
    _assert_close(got, a, b, precision)


@pytest.mark.parametrize("precision", PRECISIONS)
def test_neginf_columns_and_entries(precision):
    g = torch.Generator().manual_seed(3)
    R, I, J, K = 3, 140, 70, 300
    a = torch.rand(R, I, J, generator=g)
    b = torch.randn(R, J, K, generator=g) * 40.0
    b[0, :, 17] = float("-inf")         # whole column
    b[1, :, 0] = float("-inf")
    b[2, :, K - 1] = float("-inf")
    b[torch.rand(R, J, K, generator=g) < 0.05] = float("-inf")  # isolated entries
    b[1, : J - 1, 40] = float("-inf")   # a column with a single finite entry
    got = _run(a, b, precision=precision)
    assert not torch.isnan(got).any()
    want = orc.lm2exp_fp64(a, b)
    assert torch.all(got[0, :, 17] == float("-inf"))
    assert torch.equal(got == float("-inf"), want == float("-inf"))
    _assert_close(got, a, b, precision, want)


@pytest.mark.parametrize("precision", PRECISIONS)
def test_huge_offsets(precision):
    g = torch.Generator().manual_seed(5)
    a = torch.rand(2, 64, 128, generator=g)
    b = torch.randn(2, 128, 96, generator=g) * 10.0 + (400.0 * torch.rand(2, 1, 96, generator=g) - 200.0) * 100.0
    got = _run(a, b, precision=precision)
    want = orc.lm2exp_fp64(a, b)
    # values reach ~2e4, where one fp32 ulp is ~2e-3: compare relatively
    assert torch.allclose(got.double(), want, rtol=3e-7 if precision == "3xtf32" else 1e-6, atol=ATOL[precision])


def test_noncontiguous_inputs_and_inputs_untouched():
    g = torch.Generator().manual_seed(11)
    a_full = torch.rand(4, 100, 2 * 52, generator=g).cuda()
    b_t = torch.randn(4, 88, 52, generator=g).cuda()
    a = a_full[:, :, ::2]              # innermost stride 2 -> copy path
    b = b_t.transpose(1, 2)            # [4, 52, 88] with innermost stride 52 -> copy path
    a_before, b_before = a.clone(), b.clone()
    import triturus_b200 as tb

    got = tb.lm2exp(a, b, precision="3xtf32")
    tb.check_status()
    assert torch.equal(a, a_before) and torch.equal(b, b_before)
    _assert_close(got.cpu(), a.cpu().contiguous(), b.cpu().contiguous(), "3xtf32")
    # strided batch / row views that already satisfy the TMA rules take the no-copy path
    big_a = torch.rand(6, 128, 64, generator=g).cuda()
    big_b = torch.randn(6, 64, 256, generator=g).cuda()
    got2 = tb.lm2exp(big_a[::2, 16:80], big_b[::2, :, 64:192], precision="3xtf32")
    tb.check_status()
    _assert_close(got2.cpu(), big_a[::2, 16:80].cpu().contiguous(), big_b[::2, :, 64:192].cpu().contiguous(), "3xtf32")


def test_global_flag_selects_precision():
    from triturus.lm2exp import lm2exp
    from triturus.utils import set_tf32_enabled

    g = torch.Generator().manual_seed(13)
    a = torch.rand(2, 130, 100, generator=g).cuda()
    b = torch.randn(2, 100, 90, generator=g).cuda()
    set_tf32_enabled(False)
    hi = lm2exp(a, b)
    set_tf32_enabled(True)
    lo = lm2exp(a, b)
    set_tf32_enabled(False)
    want = orc.lm2exp_fp64(a.cpu(), b.cpu())
    e_hi = (hi.cpu().double() - want).abs().max().item()
    e_lo = (lo.cpu().double() - want).abs().max().item()
    assert e_hi <= 1e-4 and e_lo <= 2e-3 and e_hi < e_lo


def test_torch_op_is_registered_and_deterministic():
    g = torch.Generator().manual_seed(17)
    a = torch.rand(3, 200, 64, generator=g).cuda()
    b = torch.randn(3, 64, 300, generator=g).cuda()
    x = torch.ops.triturus.lm2exp(a, b, 0, 0)
    y = torch.ops.triturus.lm2exp(a, b, 0, 0)
    assert torch.equal(x, y)
    # batch permutation equivariance, bit for bit: the result of a batch entry does not depend on
    # which CTA or tile slot computed it
    perm = torch.tensor([2, 0, 1]).cuda()
    z = torch.ops.triturus.lm2exp(a[perm].contiguous(), b[perm].contiguous(), 0, 0)
    assert torch.equal(z, x[perm])


@pytest.mark.parametrize("name", ["cfg1", "cfg2", "cfg3"])
@pytest.mark.parametrize("precision", PRECISIONS)
def test_full_size_configs(name, precision):
    """The benchmark configurations at full size: float64 oracle on a batch subset, plus shift and scale
    identities on the whole result."""
    import triturus_b200 as tb
    from triturus_b200.workloads import WORKLOADS, make_inputs

    wl = WORKLOADS[name]
    a, b = make_inputs(wl, seed=0)
    ad, bd = a.cuda(), b.cuda()
    out = tb.lm2exp(ad, bd, precision=precision)
    tb.check_status()
    assert not torch.isnan(out).any()
    rs = sorted({0, wl.dims["R"] // 2, wl.dims["R"] - 1})
    want = orc.lm2exp_fp64(a[rs], b[rs])
    res = orc.compare_logspace(out[rs].cpu(), want, ATOL[precision])
    assert res["ok"], res
    # shift identity: adding c[r,k] to every b[r,:,k] adds c[r,k] to the result
    shift = torch.linspace(-3.0, 5.0, wl.dims["K"]).view(1, 1, -1).cuda()
    out_s = tb.lm2exp(ad, bd + shift, precision=precision)
    fin = torch.isfinite(out)
    assert torch.equal(torch.isfinite(out_s), fin)
    assert (out_s - shift - out)[fin].abs().max().item() <= 2 * ATOL[precision]
    # scale identity: multiplying a by 2^k adds k*log(2) exactly in exact arithmetic
    out_2 = tb.lm2exp(ad * 4.0, bd, precision=precision)
    assert (out_2 - out - 2.0 * 0.6931471805599453)[fin].abs().max().item() <= 1e-4
    tb.check_status()


@pytest.mark.parametrize("variant", [0, 101281, 101282, 201281, 201282])
@pytest.mark.parametrize("J", [1100, 4096, 16390])
def test_long_contraction_3xtf32(J, variant):
    """Contractions longer than 1024 in 3xTF32: the accumulator is re-summed in chunks of 1024 terms with
    rounded adds, so the result stays within the 3xTF32 tolerance (the tensor core's own fp32 accumulation
    truncates and would drift low by 2.6e-4 at J = 16 K).  Pre-pass and fused-max variants, one and two row
    blocks, a ragged last chunk and a ragged last k-block."""
    g = torch.Generator().manual_seed(J)
    I = 200 if variant in (0, 101282, 201282) else 100
    a = torch.rand(2, I, J, generator=g)
    b = torch.randn(2, J, 140, generator=g)
    b[1, :, 3] = float("-inf")
    got = _run(a, b, precision="3xtf32", variant=variant)
    want = orc.lm2exp_fp64(a, b)
    assert torch.all(got[1, :, 3] == float("-inf"))
    res = orc.compare_logspace(got, want, ATOL["3xtf32"])
    assert res["ok"], res


@pytest.mark.parametrize("variant", [0, 101281, 201282])
def test_long_contraction_plain_tf32(variant):
    """Plain TF32 over more than 32 K terms runs on the kernels that re-sum their accumulator every 4096 terms, so
    the stated 2e-3 holds whatever the length of the contraction (the tensor core's truncating adds alone lose
    7.8e-4 at 64 K terms and 2.5e-3 at 256 K, on top of the operand rounding)."""
    from triturus_b200 import _native

    J = 140000
    g = torch.Generator().manual_seed(variant)
    I = 200 if variant in (0, 201282) else 100
    a = torch.rand(1, I, J, generator=g)
    b = torch.randn(1, J, 140, generator=g)
    b[0, :, 3] = float("-inf")
    assert _native.LIB.triturus_b200_lm2exp_plan(1, I, J, 140, 0, variant) % 100000 // 10 == 128
    got = _run(a, b, precision="tf32", variant=variant)
    want = orc.lm2exp_fp64(a, b)
    assert torch.all(got[0, :, 3] == float("-inf"))
    res = orc.compare_logspace(got, want, ATOL["tf32"])
    assert res["ok"], res
    # the drift alone would be ~1.7e-3 here; with the re-summation the error is the operand rounding
    assert res["max_abs_err"] < 1.2e-3, res


@pytest.mark.parametrize("variant", [0, 1281, 1282, 2561, 2562, 2564])
@pytest.mark.parametrize("precision", PRECISIONS)
def test_transposed_a_is_read_in_place(precision, variant):
    """a given as a transposed view (i contiguous, triturus/lm2exp.py:190-198 forwards any strides): the
    kernels use it as an MN-major operand without a copy; results equal those of the contiguous copy."""
    import triturus_b200 as tb
    from triturus_b200 import _native

    g = torch.Generator().manual_seed(11)
    R, I, J, K = 3, 300, 172, 530               # I a multiple of 4: the transposed view meets the TMA rules
    a_t = torch.rand(R, J, I, generator=g)      # stored [R, J, I]
    b = torch.randn(R, J, K, generator=g) * 5.0 + 100.0 * torch.randn(R, 1, K, generator=g)
    a_view = a_t.cuda().transpose(1, 2)         # logical [R, I, J], stride 1 along i
    assert _native._lm2exp_a_operand(a_view, K).data_ptr() == a_view.data_ptr()
    got = tb.lm2exp(a_view, b.cuda(), precision=precision, variant=variant)
    ref = tb.lm2exp(a_view.contiguous(), b.cuda(), precision=precision, variant=variant)
    tb.check_status()
    _assert_close(got.cpu(), a_t.transpose(1, 2).contiguous(), b, precision)
    assert torch.equal(got, ref)                # same operand values in the same order


def test_transposed_a_with_odd_rows_falls_back_to_a_copy():
    import triturus_b200 as tb

    g = torch.Generator().manual_seed(12)
    a_t = torch.rand(2, 40, 131, generator=g)   # I = 131: the j stride of the view is not a multiple of 4
    b = torch.randn(2, 40, 64, generator=g)
    got = tb.lm2exp(a_t.cuda().transpose(1, 2), b.cuda(), precision="3xtf32")
    tb.check_status()
    _assert_close(got.cpu(), a_t.transpose(1, 2).contiguous(), b, "3xtf32")


@pytest.mark.parametrize("variant", [0, 1281, 1282, 2561, 2562, 101282])
@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("shape", [(2, 130, 100, 260), (3, 257, 36, 516), (1, 64, 1028, 130), (2, 7, 64, 5),
                                   (4, 512, 512, 512)])
def test_transposed_b_is_read_in_place(shape, precision, variant):
    """b given as a transposed view (j contiguous, e.g. the transpose of a contiguous [R, K, J] tensor;
    triturus/lm2exp.py:190-198 forwards any strides): the single-CTA kernel uses it as a K-major operand without a
    copy, with the row maxima of the stored tensor as stabiliser.  Ragged shapes, isolated -inf entries and an
    all -inf column."""
    import triturus_b200 as tb
    from triturus_b200 import _native

    R, I, J, K = shape
    g = torch.Generator().manual_seed(sum(shape) + variant)
    a = torch.rand(R, I, J, generator=g)
    b_t = torch.randn(R, K, J, generator=g) * 6.0 + 50.0 * torch.randn(R, K, 1, generator=g)  # stored [R, K, J]
    b_t[0, min(3, K - 1), :] = float("-inf")
    b_t[torch.rand(R, K, J, generator=g) < 0.01] = float("-inf")
    b_view = b_t.cuda().transpose(1, 2)  # logical [R, J, K], stride 1 along j
    assert _native._lm2exp_b_operand(b_view, variant).data_ptr() == b_view.data_ptr()
    got = tb.lm2exp(a.cuda(), b_view, precision=precision, variant=variant)
    tb.check_status()
    assert torch.all(got[0, :, min(3, K - 1)] == float("-inf"))
    _assert_close(got.cpu(), a, b_t.transpose(1, 2).contiguous(), precision)


def test_transposed_b_special_cases():
    """A pair tile or the fused max pass asked for by variant code, or a j extent that is not a multiple of 4
    (the k stride of the view then breaks the tensor-map rules): the wrapper makes the copy; the C ABI refuses the
    combination it cannot run.  Both operands transposed at once work in place."""
    import triturus_b200 as tb
    from triturus_b200 import _native

    g = torch.Generator().manual_seed(13)
    a = torch.rand(2, 300, 64, generator=g)
    b_t = torch.randn(2, 520, 64, generator=g) * 4.0
    b_view = b_t.cuda().transpose(1, 2)
    for variant in (2564, 202561):
        assert _native._lm2exp_b_operand(b_view, variant).data_ptr() != b_view.data_ptr()
        got = tb.lm2exp(a.cuda(), b_view, precision="tf32", variant=variant)
        tb.check_status()
        _assert_close(got.cpu(), a, b_t.transpose(1, 2).contiguous(), "tf32")
    b_odd = torch.randn(2, 130, 50, generator=g)  # J = 50
    a_odd = torch.rand(2, 40, 50, generator=g)
    got = tb.lm2exp(a_odd.cuda(), b_odd.cuda().transpose(1, 2), precision="3xtf32")
    tb.check_status()
    _assert_close(got.cpu(), a_odd, b_odd.transpose(1, 2).contiguous(), "3xtf32")
    a_t = torch.rand(2, 64, 300, generator=g)  # stored [R, J, I]
    got = tb.lm2exp(a_t.cuda().transpose(1, 2), b_view, precision="3xtf32")
    tb.check_status()
    _assert_close(got.cpu(), a_t.transpose(1, 2).contiguous(), b_t.transpose(1, 2).contiguous(), "3xtf32")
    # C ABI: a pair tile with a K-major b is an invalid combination
    R, I, J, K = 2, 300, 64, 520
    ad, out = a.cuda(), torch.empty(R, I, K, device="cuda")
    ws = torch.zeros(R * K + 64, device="cuda")
    rc = _native.LIB.triturus_b200_lm2exp_f32(
        ad.data_ptr(), b_view.data_ptr(), out.data_ptr(), R, I, J, K, _native._i64(ad.stride()),
        _native._i64(b_view.stride()), _native._i64(out.stride()), 0, 2564, ws.data_ptr(), ws.numel() * 4, None, None)
    assert rc == -1, rc  # TRITURUS_B200_EINVAL


def _raw_lm2exp(a, b, precision, variant=0):
    """The C ABI called on the tensors as they are (no wrapper in between that could copy)."""
    from triturus_b200 import _native

    R, I, J = a.shape
    K = b.shape[2]
    out = torch.empty(R, I, K, device="cuda")
    nbytes = int(_native.LIB.triturus_b200_lm2exp_workspace_bytes(R, I, J, K))
    ws = torch.zeros(nbytes // 4 + 64, device="cuda")
    rc = _native.LIB.triturus_b200_lm2exp_f32(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), R, I, J, K, _native._i64(a.stride()), _native._i64(b.stride()),
        _native._i64(out.stride()), 0 if precision == "tf32" else 1, variant, ws.data_ptr(), nbytes,
        _native._status_word(a.device).data_ptr(), None)
    torch.cuda.synchronize()
    return rc, out


@pytest.mark.parametrize("variant", [0, 1281, 1282, 2561, 101282, 201281, 301281])
@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("shape", [(2, 130, 101, 263), (1, 64, 33, 5), (3, 257, 250, 517), (2, 100, 7, 1030),
                                   (1, 300, 1026, 130)])
def test_operands_that_break_the_tensor_map_rules_are_read_in_place(shape, precision, variant):
    """Odd extents everywhere (rows of a and b that do not start on 16-byte boundaries; the reference forwards any
    strides, triturus/lm2exp.py:190-198): the C ABI takes the tensors as they are and the single-CTA kernel
    fetches them element by element.  Several tiles per CTA, partial tiles on every edge, -inf entries and an all
    -inf column; pre-pass, fused and optimistic max pass."""
    import triturus_b200 as tb

    if precision == "3xtf32" and variant % 100000 == 2561:
        pytest.skip("3xTF32 tiles have 128 columns")
    R, I, J, K = shape
    g = torch.Generator().manual_seed(sum(shape) + variant)
    a = torch.rand(R, I, J, generator=g)
    b = torch.randn(R, J, K, generator=g) * 6.0 + 50.0 * torch.randn(R, 1, K, generator=g)
    b[0, :, min(3, K - 1)] = float("-inf")
    b[torch.rand(R, J, K, generator=g) < 0.01] = float("-inf")
    rc, got = _raw_lm2exp(a.cuda(), b.cuda(), precision, variant)
    assert rc == 0, rc
    tb.check_status()
    assert torch.all(got[0, :, min(3, K - 1)] == float("-inf"))
    _assert_close(got.cpu(), a, b, precision)


@pytest.mark.parametrize("precision", PRECISIONS)
def test_strided_and_broadcast_views_in_place(precision):
    """Every third row and every second column of a, every second column of b, a b broadcast over the batch
    (stride 0) and a base that is only 4-byte aligned: through the wrapper, which for problems of this size makes
    no copy, and through the C ABI; a pair tile asked for with such operands is refused by the C ABI."""
    import triturus_b200 as tb
    from triturus_b200 import _native

    g = torch.Generator().manual_seed(21)
    a_full = torch.rand(2, 3 * 70, 2 * 48 + 1, generator=g).cuda()
    b_full = (torch.randn(2, 48, 2 * 200 + 2, generator=g) * 4.0).cuda()
    a_v, b_v = a_full[:, ::3, 1::2], b_full[:, :, 1::2][:, :, :200]
    flop = 2.0 * 2 * 70 * 48 * 200
    assert _native._in_place_small(a_v, flop, 0, False)
    assert _native._lm2exp_b_operand(b_v, 0, flop).data_ptr() == b_v.data_ptr()
    got = tb.lm2exp(a_v, b_v, precision=precision)
    tb.check_status()
    _assert_close(got.cpu(), a_v.cpu().contiguous(), b_v.cpu().contiguous(), precision)
    b_b = (torch.randn(1, 48, 200, generator=g) * 3.0).cuda().expand(2, 48, 200)
    rc, got = _raw_lm2exp(a_v, b_b, precision)
    assert rc == 0
    tb.check_status()
    _assert_close(got.cpu(), a_v.cpu().contiguous(), b_b.cpu().contiguous(), precision)
    rc, _ = _raw_lm2exp(a_v, b_v, "tf32", 2564)
    assert rc == -1  # TRITURUS_B200_EINVAL
    # a large problem with an odd extent still gets the padded copy from the wrapper (faster there)
    big = torch.rand(32, 1024, 1022, device="cuda")
    assert not _native._in_place_small(big, 2.0 * 32 * 1024 * 1022 * 1024, 0, False)


def test_batches_beyond_the_grid_limit():
    """More than 65535 batch entries (the reference's 1-D grid takes any batch, triturus/lm2exp.py:177-181): the
    library runs them in blocks of 65535 on the same stream."""
    import triturus_b200 as tb

    g = torch.Generator().manual_seed(70001)
    R = 70001
    a = torch.rand(R, 3, 5, generator=g)
    b = torch.randn(R, 5, 8, generator=g) * 4.0
    b[R - 1, :, 2] = float("-inf")
    for variant in (0, 100000):  # fused max pass; pre-pass through the workspace
        got = tb.lm2exp(a.cuda(), b.cuda(), precision="3xtf32", variant=variant)
        tb.check_status()
        _assert_close(got.cpu(), a, b, "3xtf32")
    assert torch.equal(tb.colmax(b.cuda()).cpu(), b.amax(dim=1).clamp(-1e38, 1e38))

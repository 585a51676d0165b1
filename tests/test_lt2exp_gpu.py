"""GPU parity tests for lt2exp (through the C ABI): golden fixtures from the reference's baselines, the
float64 oracle, edge cases and full-size properties.  Tolerances as in test_lm2exp_gpu.py."""

import pytest
import torch

from conftest import ATOL, LT_GOLDEN, load_golden
from oracle import logspace_oracle as orc

pytestmark = pytest.mark.gpu

PRECISIONS = ["tf32", "3xtf32"]
VARIANTS = [0, 1281, 1282, 2561, 2562, 1283, 1284, 1285]  # 1283 / 1284: generated operand in TMEM (TF32 only)


def _run(w, a, b, **kw):
    import triturus_b200 as tb

    out = tb.lt2exp(w.cuda(), a.cuda(), b.cuda(), **kw)
    tb.check_status()
    return out.cpu()


def _assert_close(got, w, a, b, precision, want64=None):
    want64 = orc.lt2exp_fp64(w, a, b, chunk=2) if want64 is None else want64
    res = orc.compare_logspace(got, want64, ATOL[precision])
    assert res["ok"], res


@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("name", LT_GOLDEN)
def test_golden(name, precision):
    g = load_golden(name)
    got = _run(g["w"], g["a"], g["b"], precision=precision)
    res = orc.compare_logspace(got, g["out"], ATOL[precision] + 2e-5)
    assert res["ok"], res
    _assert_close(got, g["w"], g["a"], g["b"], precision)


@pytest.mark.parametrize("mode", ["auto", "split", "unsplit"])
def test_modes_agree(mode):
    """The reference's three modes (triturus/lt2exp.py:533-541).  "unsplit" is one deterministic kernel; a
    split contraction adds its slices with fp32 reductions, so it agrees to rounding, not to the bit."""
    g = load_golden("lt_reftest")
    got = _run(g["w"], g["a"], g["b"], mode=mode, precision="3xtf32")
    base = _run(g["w"], g["a"], g["b"], mode="unsplit", precision="3xtf32")
    again = _run(g["w"], g["a"], g["b"], mode="unsplit", precision="3xtf32")
    assert torch.equal(base, again)
    _assert_close(got, g["w"], g["a"], g["b"], "3xtf32")
    assert (got - base).abs().max().item() <= ATOL["3xtf32"]


def test_deterministic_algorithms_switch_off_the_split():
    """ensure_reproducibility(determinism=True) (triturus/utils.py:12-31) must give run-to-run identical bits."""
    g = load_golden("lt_reftest")
    base = _run(g["w"], g["a"], g["b"], mode="unsplit", precision="3xtf32")
    torch.use_deterministic_algorithms(True, warn_only=True)
    try:
        got = _run(g["w"], g["a"], g["b"], mode="auto", precision="3xtf32")
    finally:
        torch.use_deterministic_algorithms(False)
    assert torch.equal(got, base)


SPLITS = [2, 3, 7, 16, 64, 9998, 9999]  # 9998: the tiles of the last wave shared among all SMs


@pytest.mark.parametrize("split", SPLITS)
@pytest.mark.parametrize("tile", [0, 1281, 2562, 1283, 1284, 1285])
@pytest.mark.parametrize("precision", PRECISIONS)
def test_contraction_split(precision, tile, split):
    """Explicit slice counts on a ragged shape: I not divisible by the slice count, J not a multiple of the
    32-wide chunk, -inf entries and one all -inf column."""
    if precision == "3xtf32" and tile in (2562, 1283, 1284, 1285):
        pytest.skip("no 256 x 256 tile and no TMEM-operand kernel in 3xTF32")
    g = torch.Generator().manual_seed(100 + split)
    R, S, I, J, K = 2, 150, 37, 70, 140
    w = torch.rand(R, S, I, J, generator=g)
    a = torch.randn(R, I, K, generator=g) * 6.0
    b = torch.randn(R, J, K, generator=g) * 6.0 - 20.0
    a[torch.rand(R, I, K, generator=g) < 0.03] = float("-inf")
    b[1, :, 11] = float("-inf")
    got = _run(w, a, b, precision=precision, variant=split * 10000 + tile)
    want = orc.lt2exp_fp64(w, a, b)
    assert not torch.isnan(got).any()
    assert torch.all(got[1, :, 11] == float("-inf"))
    assert torch.equal(got == float("-inf"), want == float("-inf"))
    _assert_close(got, w, a, b, precision, want)


def test_contraction_split_strided_output_rows_untouched():
    """The zero-fill and log passes of a split launch follow the output strides: padding between the rows of
    a strided result keeps its contents."""
    import ctypes

    from triturus_b200 import _native

    g = torch.Generator().manual_seed(5)
    R, S, I, J, K = 2, 40, 24, 64, 72
    w = torch.rand(R, S, I, J, generator=g).cuda()
    a = torch.randn(R, I, K, generator=g).cuda()
    b = torch.randn(R, J, K, generator=g).cuda()
    buf = torch.full((R, S, K + 8), 7.0, device="cuda")
    out = buf[:, :, :K]
    i64 = ctypes.c_int64
    rc = _native.LIB.triturus_b200_lt2exp_f32(
        w.data_ptr(), a.data_ptr(), b.data_ptr(), out.data_ptr(), R, S, I, J, K,
        (i64 * 4)(*w.stride()), (i64 * 3)(*a.stride()), (i64 * 3)(*b.stride()), (i64 * 3)(*out.stride()),
        1, 8 * 10000, _native._status_word(w.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    _native.check_status()
    assert _native.LIB.triturus_b200_lt2exp_launches(R, S, I, J, K, 1, 8 * 10000) == 3
    assert _native.LIB.triturus_b200_lt2exp_launches(R, S, I, J, K, 1, 1 * 10000) == 1
    assert torch.all(buf[:, :, K:] == 7.0)
    _assert_close(out.cpu(), w.cpu(), a.cpu(), b.cpu(), "3xtf32")


@pytest.mark.parametrize("precision", PRECISIONS)
def test_split_few_tiles_long_contraction(precision):
    """One output tile and a 128 x 128 contraction: the automatic mode spreads the slices over the SMs."""
    from triturus_b200 import _native

    g = torch.Generator().manual_seed(77)
    w = torch.rand(1, 128, 128, 128, generator=g)
    a = torch.randn(1, 128, 128, generator=g)
    b = torch.randn(1, 128, 128, generator=g)
    assert _native.LIB.triturus_b200_lt2exp_launches(1, 128, 128, 128, 128, 0, 0) == 3
    got = _run(w, a, b, precision=precision)
    _assert_close(got, w, a, b, precision)


def test_unknown_mode_raises():
    import triturus_b200 as tb

    g = load_golden("lt_neginf")
    with pytest.raises(ValueError):
        tb.lt2exp(g["w"].cuda(), g["a"].cuda(), g["b"].cuda(), mode="fast")


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("precision", PRECISIONS)
def test_variants_on_ragged_shape(precision, variant):
    if precision == "3xtf32" and variant in (1283, 1284, 1285):
        pytest.skip("the TMEM-operand kernel is TF32 only")
    g = torch.Generator().manual_seed(9)
    w = torch.rand(3, 270, 13, 37, generator=g)
    a = torch.randn(3, 13, 300, generator=g) * 4.0 + 50.0 * torch.randn(3, 1, 300, generator=g)
    b = torch.randn(3, 37, 300, generator=g) * 4.0
    got = _run(w, a, b, precision=precision, variant=variant)
    _assert_close(got, w, a, b, precision)


@pytest.mark.parametrize("shape", [(1, 1, 1, 1, 1), (1, 3, 1, 33, 5), (2, 129, 5, 1, 3), (2, 7, 9, 64, 257),
                                   (1, 130, 20, 31, 70), (2, 128, 4, 32, 128), (1, 64, 17, 96, 258)])
@pytest.mark.parametrize("precision", PRECISIONS)
def test_edge_shapes(shape, precision):
    R, S, I, J, K = shape
    g = torch.Generator().manual_seed(sum(shape))
    w = torch.rand(R, S, I, J, generator=g) + 0.01
    a = torch.randn(R, I, K, generator=g) * 3.0
    b = torch.randn(R, J, K, generator=g) * 3.0
    got = _run(w, a, b, precision=precision)
    assert got.shape == (R, S, K) and got.is_contiguous()
    _assert_close(got, w, a, b, precision)


@pytest.mark.parametrize("precision", PRECISIONS)
def test_neginf_columns_and_entries(precision):
    g = torch.Generator().manual_seed(4)
    R, S, I, J, K = 2, 140, 12, 40, 200
    w = torch.rand(R, S, I, J, generator=g)
    a = torch.randn(R, I, K, generator=g) * 30.0
    b = torch.randn(R, J, K, generator=g) * 30.0
    a[0, :, 7] = float("-inf")
    b[1, :, 199] = float("-inf")
    a[1, :, 50] = float("-inf")
    b[1, :, 50] = float("-inf")
    a[torch.rand(R, I, K, generator=g) < 0.05] = float("-inf")
    b[torch.rand(R, J, K, generator=g) < 0.05] = float("-inf")
    got = _run(w, a, b, precision=precision)
    assert not torch.isnan(got).any()
    want = orc.lt2exp_fp64(w, a, b)
    assert torch.all(got[0, :, 7] == float("-inf")) and torch.all(got[1, :, 50] == float("-inf"))
    assert torch.equal(got == float("-inf"), want == float("-inf"))
    _assert_close(got, w, a, b, precision, want)


def test_noncontiguous_a_b_and_w_view_contract():
    import triturus_b200 as tb

    g = torch.Generator().manual_seed(21)
    w = torch.rand(2, 40, 6, 20, generator=g).cuda()
    a_t = torch.randn(2, 90, 6, generator=g).cuda()
    b_big = torch.randn(2, 20, 180, generator=g).cuda()
    a = a_t.transpose(1, 2)        # [2, 6, 90], innermost stride 6
    b = b_big[:, :, ::2]           # [2, 20, 90], innermost stride 2
    got = tb.lt2exp(w, a, b, precision="3xtf32")
    tb.check_status()
    _assert_close(got.cpu(), w.cpu(), a.cpu().contiguous(), b.cpu().contiguous(), "3xtf32")
    # like the reference (triturus/lt2exp.py:549), w must allow .view(R, S, -1)
    w_bad = torch.rand(2, 40, 20, 6, generator=g).cuda().transpose(2, 3)  # [2, 40, 6, 20], not viewable
    with pytest.raises(RuntimeError):
        tb.lt2exp(w_bad, a, b)


def test_batch_permutation_is_bit_exact():
    g = torch.Generator().manual_seed(23)
    w = torch.rand(3, 150, 8, 40, generator=g).cuda()
    a = torch.randn(3, 8, 260, generator=g).cuda()
    b = torch.randn(3, 40, 260, generator=g).cuda()
    x = torch.ops.triturus.lt2exp(w, a, b, 0, 10000)  # unsplit: the deterministic path
    perm = torch.tensor([1, 2, 0]).cuda()
    z = torch.ops.triturus.lt2exp(w[perm].contiguous(), a[perm].contiguous(), b[perm].contiguous(), 0, 10000)
    assert torch.equal(z, x[perm])


@pytest.mark.parametrize("name,batch", [("cfg4", 16), ("cfg5", 4)])
@pytest.mark.parametrize("precision", PRECISIONS)
def test_full_size_configs(name, batch, precision):
    """cfg4 at full size; cfg5 with its full S, I, J, K and four batch entries (one entry of cfg5 is
    17 G multiply-adds for the float64 oracle).  Oracle on a batch subset plus the shift identity."""
    import triturus_b200 as tb
    from triturus_b200.workloads import WORKLOADS, make_inputs

    wl = WORKLOADS[name].with_batch(batch)
    w, a, b = make_inputs(wl, seed=0)
    wd, ad, bd = w.cuda(), a.cuda(), b.cuda()
    out = tb.lt2exp(wd, ad, bd, precision=precision)
    tb.check_status()
    assert not torch.isnan(out).any()
    rs = [0, batch - 1] if name == "cfg4" else [batch - 1]
    want = orc.lt2exp_fp64(w[rs], a[rs], b[rs])
    res = orc.compare_logspace(out[rs].cpu(), want, ATOL[precision])
    assert res["ok"], res
    K = wl.dims["K"]
    sa = torch.linspace(-2.0, 3.0, K).view(1, 1, -1).cuda()
    sb = torch.linspace(4.0, -1.0, K).view(1, 1, -1).cuda()
    out_s = tb.lt2exp(wd, ad + sa, bd + sb, precision=precision)
    fin = torch.isfinite(out)
    assert torch.equal(torch.isfinite(out_s), fin)
    assert (out_s - sa - sb - out)[fin].abs().max().item() <= 2 * ATOL[precision]
    tb.check_status()


@pytest.mark.parametrize("tile", [0, 1281, 1282, 2561, 2562, 1283, 1285])
@pytest.mark.parametrize("precision", PRECISIONS)
def test_contraction_shared_last_wave(precision, tile):
    """Whole waves plus a shared last wave on a shape with several waves of tiles (256 tiles of 128 x 128 down to 32
    of 256 x 256 on 148 SMs): equal parts when the last wave is less than half full, mains and tails otherwise;
    parts start and end inside j-chunk rows (a tile's contraction is 40 k-blocks of 20 rows i x 2 j-chunks)."""
    if precision == "3xtf32" and tile in (2562, 1283, 1285):
        pytest.skip("no 256 x 256 tile and no TMEM-operand kernel in 3xTF32")
    from triturus_b200 import _native

    g = torch.Generator().manual_seed(808)
    R, S, I, J, K = 16, 256, 20, 64, 1024
    w = torch.rand(R, S, I, J, generator=g)
    a = torch.randn(R, I, K, generator=g) * 5.0
    b = torch.randn(R, J, K, generator=g) * 5.0 - 30.0
    b[torch.rand(R, J, K, generator=g) < 0.02] = float("-inf")
    a[3, :, 77] = float("-inf")
    variant = 9998 * 10000 + tile
    prec = 0 if precision == "tf32" else 1
    # With scratch memory (what the Python wrapper passes) the kernels that build their operand in shared memory
    # complete shared tiles in the same launch; the TMEM-operand kernels add into the zero-filled result.
    tmem_tile = _native.LIB.triturus_b200_lt2exp_plan(R, S, I, J, K, prec, variant) % 10000 in (1283, 1284, 1285)
    assert _native.LIB.triturus_b200_lt2exp_launches(R, S, I, J, K, prec, variant) == (3 if tmem_tile else 1)
    assert (_native.LIB.triturus_b200_lt2exp_workspace_bytes(R, S, I, J, K, prec, variant) > 0) == (not tmem_tile)
    assert _native.LIB.triturus_b200_lt2exp_plan(R, S, I, J, K, prec, variant) // 10000 == 9998
    got = _run(w, a, b, precision=precision, variant=variant)
    want = orc.lt2exp_fp64(w, a, b)
    assert torch.all(got[3, :, 77] == float("-inf"))
    assert torch.equal(got == float("-inf"), want == float("-inf"))
    _assert_close(got, w, a, b, precision, want)
    if not tmem_tile:
        # parked partial sums are added in a fixed order: a second call gives the same bits
        assert torch.equal(got, _run(w, a, b, precision=precision, variant=variant))
        # the entry point without scratch memory runs the same ranges with additions into the result
        import ctypes

        wd, ad, bd = w.cuda(), a.cuda(), b.cuda()
        out = torch.empty((R, S, K), device="cuda")
        i64 = ctypes.c_int64
        rc = _native.LIB.triturus_b200_lt2exp_f32(
            wd.data_ptr(), ad.data_ptr(), bd.data_ptr(), out.data_ptr(), R, S, I, J, K,
            (i64 * 4)(*wd.stride()), (i64 * 3)(*ad.stride()), (i64 * 3)(*bd.stride()), (i64 * 3)(*out.stride()),
            prec, variant, _native._status_word(wd.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        _native.check_status()
        _assert_close(out.cpu(), w, a, b, precision, want)


def test_automatic_choice_balances_a_ragged_last_wave():
    """R = 8 entries of cfg5's shape are 128 tiles of 256 x 256 on 148 SMs: the automatic choice shares the
    contractions of that last (only) wave among all SMs; the full R = 64 (6.9 waves) and a deterministic call keep
    whole tiles."""
    from triturus_b200 import _native

    plan = _native.LIB.triturus_b200_lt2exp_plan
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    if sms != 148:
        pytest.skip("the tile counts in this test are for 148 SMs")
    assert plan(8, 256, 128, 128, 4096, 0, 0) == 9998 * 10000 + 2562
    assert plan(64, 256, 128, 128, 4096, 0, 0) == 1 * 10000 + 2562
    assert plan(8, 256, 128, 128, 4096, 0, 1 * 10000) == 1 * 10000 + 2562
    # cfg4: a tile's contraction (128 k-blocks) is too short to pay for the two extra launches
    assert plan(16, 128, 64, 64, 2048, 0, 0) == 1 * 10000 + 1285


@pytest.mark.parametrize("variant", [1 * 10000 + 2562, 9998 * 10000 + 2562])
@pytest.mark.parametrize("precision", PRECISIONS)
def test_cfg5_on_the_benchmarked_tile(precision, variant):
    """cfg5's own distribution (N(-40, 15), 0.5 % -inf, I * J = 16384) on the tile the benchmarks run: 256 x 256
    as whole tiles (12562, what the full R = 64 runs on one GPU) and with the last wave shared (99982562,
    what R = 64 / N runs per GPU on 2, 4 and 8 GPUs).  The float64 oracle checks one batch entry; the whole
    result is checked for NaN, for its -inf positions and with the shift identity."""
    import triturus_b200 as tb
    from triturus_b200 import _native
    from triturus_b200.workloads import WORKLOADS, make_inputs

    R = 16
    wl = WORKLOADS["cfg5"].with_batch(R)
    d = wl.dims
    prec = 0 if precision == "tf32" else 1
    if precision == "tf32" and torch.cuda.get_device_properties(0).multi_processor_count == 148:
        # what bench.py runs at R = 64 (one GPU) and at R = 8 (eight GPUs) is what this test pins
        plan = _native.LIB.triturus_b200_lt2exp_plan
        assert plan(64, d["S"], d["I"], d["J"], d["K"], prec, 0) == 12562
        assert plan(8, d["S"], d["I"], d["J"], d["K"], prec, 0) == 99982562
    w, a, b = make_inputs(wl, seed=0)
    wd, ad, bd = w.cuda(), a.cuda(), b.cuda()
    out = tb.lt2exp(wd, ad, bd, precision=precision, variant=variant)
    auto = tb.lt2exp(wd, ad, bd, precision=precision)
    tb.check_status()
    assert not torch.isnan(out).any()
    # a result is -inf exactly where a whole column of a or of b is -inf (w > 0 everywhere)
    dead = (torch.isinf(ad).all(dim=1) | torch.isinf(bd).all(dim=1)).unsqueeze(1).expand_as(out)
    assert torch.equal(out == float("-inf"), dead)
    assert torch.equal(torch.isinf(auto), torch.isinf(out))
    r = R - 3
    want = orc.lt2exp_fp64(w[r : r + 1], a[r : r + 1], b[r : r + 1])
    res = orc.compare_logspace(out[r : r + 1].cpu(), want, ATOL[precision])
    assert res["ok"], res
    # every other batch entry against the automatic tile choice (checked above on its own merits)
    fin = torch.isfinite(out)
    assert (out - auto)[fin].abs().max().item() <= 2 * ATOL[precision]
    K = d["K"]
    sa = torch.linspace(-2.0, 3.0, K).view(1, 1, -1).cuda()
    sb = torch.linspace(4.0, -1.0, K).view(1, 1, -1).cuda()
    out_s = tb.lt2exp(wd, ad + sa, bd + sb, precision=precision, variant=variant)
    assert torch.equal(torch.isfinite(out_s), fin)
    assert (out_s - sa - sb - out)[fin].abs().max().item() <= 2 * ATOL[precision]
    tb.check_status()


@pytest.mark.parametrize("variant", [1283, 1284, 1285])
@pytest.mark.parametrize("shape", [(1, 1, 1, 1, 1), (2, 129, 5, 1, 3), (2, 7, 9, 64, 257), (1, 300, 20, 31, 70),
                                   (3, 256, 16, 40, 384)])
def test_tmem_operand_kernel_edge_shapes(shape, variant):
    """The transposed kernel (operand in TMEM) on ragged shapes, with -inf entries and an all -inf column."""
    R, S, I, J, K = shape
    g = torch.Generator().manual_seed(sum(shape) + variant)
    w = torch.rand(R, S, I, J, generator=g) + 0.01
    a = torch.randn(R, I, K, generator=g) * 3.0
    b = torch.randn(R, J, K, generator=g) * 3.0 - 10.0
    a[torch.rand(R, I, K, generator=g) < 0.05] = float("-inf")
    b[R - 1, :, K - 1] = float("-inf")
    got = _run(w, a, b, precision="tf32", variant=variant)
    want = orc.lt2exp_fp64(w, a, b)
    assert not torch.isnan(got).any()
    assert torch.equal(got == float("-inf"), want == float("-inf"))
    _assert_close(got, w, a, b, "tf32", want)


def test_tmem_operand_kernel_refuses_3xtf32():
    import triturus_b200 as tb

    w = torch.rand(1, 8, 4, 4).cuda()
    a = torch.randn(1, 4, 8).cuda()
    with pytest.raises(tb.NativeLibraryError):
        tb.lt2exp(w, a, a.clone(), precision="3xtf32", variant=1283)


@pytest.mark.parametrize("variant", [8 * 10000, 8 * 10000 + 1283])
@pytest.mark.parametrize("precision", PRECISIONS)
def test_contraction_split_odd_columns(precision, variant):
    """K not a multiple of 4: the column maxima (main kernel and log pass) take the scalar path and the slices
    add with scalar reductions."""
    if precision == "3xtf32" and variant % 10000 == 1283:
        pytest.skip("the TMEM-operand kernel is TF32 only")
    g = torch.Generator().manual_seed(55)
    R, S, I, J, K = 2, 70, 40, 50, 141
    w = torch.rand(R, S, I, J, generator=g)
    a = torch.randn(R, I, K, generator=g) * 4.0
    b = torch.randn(R, J, K, generator=g) * 4.0
    b[0, :, 140] = float("-inf")
    got = _run(w, a, b, precision=precision, variant=variant)
    want = orc.lt2exp_fp64(w, a, b)
    assert torch.all(got[0, :, 140] == float("-inf"))
    _assert_close(got, w, a, b, precision, want)


def test_batches_beyond_the_grid_limit():
    """More than 65535 batch entries run in blocks of 65535 on the same stream (whole tiles and split contraction)."""
    g = torch.Generator().manual_seed(66000)
    R = 66000
    w = torch.rand(R, 2, 3, 4, generator=g)
    a = torch.randn(R, 3, 8, generator=g) * 3.0
    b = torch.randn(R, 4, 8, generator=g) * 3.0
    a[R - 1, :, 1] = float("-inf")
    for variant in (10000, 2 * 10000):
        got = _run(w, a, b, precision="3xtf32", variant=variant)
        _assert_close(got, w, a, b, "3xtf32")


@pytest.mark.parametrize("variant", [0, 11281, 11282, 12561, 11283, 11285, 99981281])
@pytest.mark.parametrize("precision", ["tf32", "3xtf32"])
def test_strided_views_of_a_and_b_are_read_in_place(precision, variant):
    """a and b as transposed views (k stride = I resp. J), as every second column of a wider tensor, and broadcast over
    the batch (stride 0): the reference forwards any strides (triturus/lt2exp.py:580-585, :612-617) and so does the
    C ABI; no copy is made on the way."""
    import triturus_b200 as tb

    if precision == "3xtf32" and variant in (12561, 11283, 11285):
        pytest.skip("tile not available in 3xTF32")
    g = torch.Generator().manual_seed(31 + variant)
    R, S, I, J, K = 3, 70, 12, 20, 300
    w = torch.rand(R, S, I, J, generator=g)
    a_t = (torch.randn(R, K, I, generator=g) * 3.0).cuda()      # stored [R, K, I]
    b_wide = (torch.randn(R, J, 2 * K + 1, generator=g) * 3.0).cuda()
    a_v, b_v = a_t.transpose(1, 2), b_wide[:, :, 1::2][:, :, :K]
    a_v[0, :, 5] = float("-inf")
    got = tb.lt2exp(w.cuda(), a_v, b_v, precision=precision, variant=variant)
    tb.check_status()
    want = orc.lt2exp_fp64(w, a_v.cpu().contiguous(), b_v.cpu().contiguous())
    res = orc.compare_logspace(got.cpu(), want, ATOL[precision])
    assert res["ok"], res
    assert torch.all(got[0, :, 5] == float("-inf"))
    b_b = (torch.randn(1, J, K, generator=g) * 3.0).cuda().expand(R, J, K)  # the same b for every batch entry
    got = tb.lt2exp(w.cuda(), a_v, b_b, precision=precision, variant=variant)
    tb.check_status()
    res = orc.compare_logspace(got.cpu(), orc.lt2exp_fp64(w, a_v.cpu().contiguous(), b_b.cpu().contiguous()), ATOL[precision])
    assert res["ok"], res

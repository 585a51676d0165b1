"""CPU: the C-ABI library loads and exports what include/triturus_b200.h declares; the Python wrappers keep
the reference's argument checks; nothing here launches a kernel."""

import ctypes
import re
from pathlib import Path

import pytest
import torch

import triturus_b200
from triturus_b200 import _native
from triturus_b200 import build as tb_build

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "triturus_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(triturus_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    names = _declared_symbols()
    assert "triturus_b200_lm2exp_f32" in names and "triturus_b200_lt2exp_f32" in names
    lib = ctypes.CDLL(str(tb_build.LIB_PATH))
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    for n in _native.EXPORTED_SYMBOLS:
        assert n in names, f"{n} bound in Python but not declared in the header"


def test_version_and_strerror():
    assert _native.LIB.triturus_b200_version() >= 100
    assert _native.strerror(0) == "ok"
    assert "align" in _native.strerror(-2)
    assert "timed out" in _native.strerror(103)


def test_workspace_bytes():
    f = _native.LIB.triturus_b200_lm2exp_workspace_bytes
    # 256 bytes for the flag words of the optimistic stabiliser, then R x K stabilisers
    assert f(32, 1024, 1024, 1024) == 256 + 32 * 1024 * 4
    assert f(3, 7, 5, 11) == 256 + 3 * 11 * 4
    assert f(0, 1, 1, 1) == 0


def test_argument_validation_returns_codes_without_a_gpu():
    """Bad arguments are rejected before any CUDA call, so these run on a CPU-only machine."""
    lib = _native.LIB
    s3 = _native._i64([12, 4, 1])
    null = ctypes.c_void_p(0)
    fake = ctypes.c_void_p(4096)
    fake2 = ctypes.c_void_p(8192)
    chain = lib.triturus_b200_lm2exp_chain_f32
    rc = lib.triturus_b200_lm2exp_f32(null, fake, fake, 1, 1, 4, 4, s3, s3, s3, 0, 0, fake, 1 << 20, null, null)
    assert rc == -1  # NULL operand
    rc = lib.triturus_b200_lm2exp_f32(fake, fake, fake, 1, 0, 4, 4, s3, s3, s3, 0, 0, fake, 1 << 20, null, null)
    assert rc == -1  # empty dimension
    rc = lib.triturus_b200_lm2exp_f32(fake, fake, fake, 1, 1, 4, 4, s3, s3, s3, 7, 0, fake, 1 << 20, null, null)
    assert rc == -1  # unknown precision
    rc = lib.triturus_b200_lm2exp_f32(fake, fake, fake, 1, 1, 4, 4, s3, s3, s3, 0, 0, fake, 8, null, null)
    assert rc == -3  # workspace too small
    # (operands a and b may have any strides; the result must have innermost stride 1, and fp32 data is 4-byte aligned)
    bad = _native._i64([12, 4, 2])
    rc = lib.triturus_b200_lm2exp_f32(fake, fake, fake, 1, 1, 4, 4, s3, s3, bad, 0, 0, fake, 1 << 20, null, null)
    assert rc == -2  # innermost stride of the result must be 1
    rc = lib.triturus_b200_lm2exp_f32(ctypes.c_void_p(4098), fake, fake, 1, 1, 4, 4, s3, s3, s3, 0, 0, fake, 1 << 20, null, null)
    assert rc == -2  # operand not 4-byte aligned
    odd = _native._i64([14, 7, 1])
    rc = lib.triturus_b200_lm2exp_f32(fake, fake, fake, 2, 2, 4, 4, odd, s3, s3, 0, 2564, fake, 1 << 20, null, null)
    assert rc == -1  # a row stride that is not a multiple of 4 elements cannot go with a pair tile
    rc = chain(fake, fake, fake, 2, 2, 4, 4, odd, s3, s3, 0, 0, fake, fake2, fake, 1 << 20, null, null)
    assert rc == -2  # ... nor with returned column maxima
    s4 = _native._i64([48, 16, 4, 1])
    rc = lib.triturus_b200_lt2exp_f32(fake, fake, fake, null, 1, 1, 4, 4, 4, s4, s3, s3, s3, 0, 0, null, null)
    assert rc == -1
    rc = lib.triturus_b200_lt2exp_f32(fake, fake, fake, fake, 1, 1, 4, 4, 4, s4, s3, s3, s3, 0, 5, null, null)
    assert rc == -1  # unknown variant
    # chain entry point: no workspace and no stabiliser; the same buffer for both sets of maxima; a fused
    # max pass requested together with a supplied stabiliser
    chain = lib.triturus_b200_lm2exp_chain_f32
    rc = chain(fake, fake, fake, 1, 1, 4, 4, s3, s3, s3, 0, 0, null, null, null, 0, null, null)
    assert rc == -3
    rc = chain(fake, fake, fake, 1, 1, 4, 4, s3, s3, s3, 0, 0, fake, fake, null, 0, null, null)
    assert rc == -1
    rc = chain(fake, fake, fake, 1, 1, 4, 4, s3, s3, s3, 0, 201281, fake, null, null, 0, null, null)
    assert rc == -1
    # lt2exp chain entry point: one set of maxima without the other; the same buffer in and out
    ltc = lib.triturus_b200_lt2exp_chain_f32
    rc = ltc(fake, fake, fake, fake, 1, 1, 4, 4, 4, s4, s3, s3, s3, 0, 0, fake, null, null, null, null)
    assert rc == -1
    rc = ltc(fake, fake, fake, fake, 1, 1, 4, 4, 4, s4, s3, s3, s3, 0, 0, fake, fake, fake, null, null)
    assert rc == -1


def test_wrappers_keep_reference_assertions():
    from triturus.lm2exp import lm2exp
    from triturus.lt2exp import lt2exp

    with pytest.raises(AssertionError):
        lm2exp(torch.rand(2, 3), torch.rand(2, 3, 4))
    with pytest.raises(AssertionError):
        lm2exp(torch.rand(2, 3, 4), torch.rand(3, 4, 5))
    with pytest.raises(AssertionError):
        lm2exp(torch.rand(2, 3, 4), torch.rand(2, 5, 5))
    with pytest.raises(AssertionError):
        lm2exp(torch.rand(2, 3, 4).double(), torch.rand(2, 4, 5).double())
    with pytest.raises(AssertionError):
        lt2exp(torch.rand(2, 3, 4, 5), torch.rand(2, 4, 6), torch.rand(2, 4, 6))
    with pytest.raises(AssertionError):
        lt2exp(torch.rand(2, 3, 4), torch.rand(2, 4, 6), torch.rand(2, 5, 6))
    with pytest.raises(ValueError):
        lt2exp(torch.rand(2, 3, 4, 5), torch.rand(2, 4, 6), torch.rand(2, 5, 6), mode="bogus")


def test_no_cpu_fallback():
    """CPU tensors are refused: the product path is the CUDA library only."""
    with pytest.raises(triturus_b200.NativeLibraryError):
        triturus_b200.lm2exp(torch.rand(2, 3, 4), torch.rand(2, 4, 5))
    with pytest.raises(triturus_b200.NativeLibraryError):
        triturus_b200.lt2exp(torch.rand(2, 3, 4, 5), torch.rand(2, 4, 6), torch.rand(2, 5, 6))


def test_precision_flag_mapping():
    from triturus.utils import is_triturus_tf32_enabled, set_tf32_enabled
    from triturus_b200.utils import resolve_precision

    assert not is_triturus_tf32_enabled() and resolve_precision(None) == 1
    set_tf32_enabled(True)
    assert is_triturus_tf32_enabled() and resolve_precision(None) == 0
    assert torch.backends.cuda.matmul.allow_tf32
    set_tf32_enabled(False)
    assert resolve_precision("tf32") == 0 and resolve_precision("3xtf32") == 1
    with pytest.raises(ValueError):
        resolve_precision("fp16")


def test_chain_launch_counts():
    """Kernels per call of the chain entry point: a supplied stabiliser removes the pre-pass (or turns the
    fused max pass off), returned column maxima add one fill launch."""
    f = _native.LIB.triturus_b200_lm2exp_chain_launches
    assert f(32, 1024, 1024, 1024, 0, 0, 0, 0) == _native.LIB.triturus_b200_lm2exp_launches(32, 1024, 1024, 1024, 0, 0)
    assert f(32, 1024, 1024, 1024, 0, 0, 1, 0) == 1
    assert f(32, 1024, 1024, 1024, 0, 0, 1, 1) == 2
    assert f(256, 128, 256, 8192, 1, 0, 0, 0) == 1  # fused max pass
    assert f(256, 128, 256, 8192, 0, 0, 0, 0) == 2  # plain TF32: optimistic max pass + conditional launch of the full one
    assert f(256, 128, 256, 8192, 0, 0, 0, 1) == 1  # returned column maxima: exact pass
    assert f(128, 256, 256, 8192, 0, 0, 1, 1) == 1  # one row tile: maxima stored directly, no fill
    assert f(32, 1024, 1024, 1024, 0, 202561, 1, 0) < 0


def test_fake_kernels_infer_shapes():
    a = torch.empty(3, 5, 7, device="meta")
    b = torch.empty(3, 7, 9, device="meta")
    assert torch.ops.triturus.lm2exp(a, b, 0, 0).shape == (3, 5, 9)
    w = torch.empty(3, 4, 5, 7, device="meta")
    a = torch.empty(3, 5, 9, device="meta")
    assert torch.ops.triturus.lt2exp(w, a, b, 1, 0).shape == (3, 4, 9)
    a = torch.empty(3, 5, 7, device="meta")
    out, m = torch.ops.triturus.lm2exp_chain(a, b, None, True, 0, 0)
    assert out.shape == (3, 5, 9) and m.shape == (3, 9)
    out, m = torch.ops.triturus.lm2exp_chain(a, b, torch.empty(3, 9, device="meta"), False, 0, 0)
    assert out.shape == (3, 5, 9) and m.numel() == 0
    a = torch.empty(3, 5, 9, device="meta")
    out, m = torch.ops.triturus.lt2exp_chain(w, a, b, None, None, True, 0, 0)
    assert out.shape == (3, 4, 9) and m.shape == (3, 9)


def test_tma_ready_padding_rules():
    t = torch.rand(2, 3, 50)
    v = _native._tma_ready(t)
    assert v.shape == t.shape and v.stride(-1) == 1 and v.stride(1) % 4 == 0 and torch.equal(v, t)
    t2 = torch.rand(2, 3, 48)
    assert _native._tma_ready(t2) is t2
    t3 = torch.rand(2, 48, 3).transpose(1, 2)
    v3 = _native._tma_ready(t3)
    assert v3.stride(-1) == 1 and torch.equal(v3, t3)


def test_transposed_a_is_kept_or_copied_by_cost():
    """A transposed view of lm2exp's a is a legal MN-major operand; the wrapper keeps it when its estimate of
    the transposing copy exceeds 16 % of its estimate of the kernel time, and copies otherwise or when the
    view breaks the TMA rules (stride not a multiple of 4 elements)."""
    view = torch.rand(2, 172, 300).transpose(1, 2)          # [2, 300, 172], i contiguous
    assert _native._lm2exp_a_operand(view, 530) is view       # a third of all bytes: in place
    assert _native._lm2exp_a_operand(view, 1 << 20) is not view  # a vanishing part of a huge problem: copy
    odd = torch.rand(2, 40, 131).transpose(1, 2)            # j stride 131: not a multiple of 4
    got = _native._lm2exp_a_operand(odd, 64)
    assert got is not odd and got.stride(2) == 1 and torch.equal(got, odd)
    plain = torch.rand(2, 300, 172)
    assert _native._lm2exp_a_operand(plain, 530) is plain


def test_workload_generators_are_seeded_and_shaped():
    from triturus_b200.workloads import WORKLOADS, make_inputs

    wl = WORKLOADS["cfg2"].with_batch(1)
    a1, b1 = make_inputs(wl, seed=0)
    a2, b2 = make_inputs(wl, seed=0)
    assert torch.equal(a1, a2) and torch.equal(b1, b2)
    assert a1.shape == (1, 1024, 1024) and b1.shape == (1, 1024, 1024)
    assert torch.isinf(b1).float().mean() > 0.005
    assert WORKLOADS["cfg2"].flops == 2.0 * 32 * 1024**3
    assert WORKLOADS["cfg5"].bytes == 4.0 * 64 * (256 * 128 * 128 + 2 * 128 * 4096 + 256 * 4096)


def test_host_pipeline_chunking():
    from triturus_b200.host import chunk_bounds

    def check(bounds, batch):
        assert bounds[0][0] == 0 and bounds[-1][1] == batch
        assert all(lo < hi for lo, hi in bounds)
        assert all(bounds[i][1] == bounds[i + 1][0] for i in range(len(bounds) - 1))
        return [hi - lo for lo, hi in bounds]

    # explicit chunk counts: equal sizes
    for batch, chunks in ((7, 3), (5, 16), (3, 1), (64, 9)):
        sizes = check(chunk_bounds(batch, 1 << 20, chunks), batch)
        assert max(sizes) - min(sizes) <= 1 and len(sizes) == min(chunks, batch)
    # automatic: ~32 MB chunks with a short ramp at both ends (cfg2: 32 entries of 8 MB -> 1, 2, 4 ... 4, 2, 1)
    sizes = check(chunk_bounds(32, 8 << 20), 32)
    assert sizes[:2] == [1, 2] and sizes[-2:] == [2, 1] and max(sizes) <= 5 and min(sizes[2:-2]) >= 3
    assert check(chunk_bounds(1, 1 << 30), 1) == [1]
    assert check(chunk_bounds(4, 1 << 10), 4) == [4]            # small problems: one chunk
    assert len(check(chunk_bounds(1000, 1 << 30), 1000)) == 16  # huge entries: one per chunk, at most 16 chunks
    for batch in (2, 3, 9, 64, 129):
        check(chunk_bounds(batch, 12 << 20), batch)
    with pytest.raises(ValueError):
        chunk_bounds(0, 4)


def test_operand_preparation_rules():
    """Which lm2exp operands the wrapper passes as they are and which it copies (pure host logic, CPU tensors)."""
    x = torch.zeros(2, 64, 96)
    assert _native._tma_ok(x)
    assert not _native._tma_ok(x[:, :, ::2])          # innermost stride 2
    assert not _native._tma_ok(torch.zeros(2, 64, 97))  # row pitch not a multiple of 4 elements
    assert _native._tma_ok(torch.zeros(1, 1, 97))     # strides of size-1 dimensions do not matter
    assert _native._tma_ready(x) is x
    padded = _native._tma_ready(torch.ones(2, 5, 7))
    assert padded.shape == (2, 5, 7) and padded.stride() == (40, 8, 1) and bool((padded == 1).all())
    # b: plain, transposed (j contiguous), odd
    b_t = torch.zeros(2, 96, 64).transpose(1, 2)      # [R, J=64, K=96] with stride 1 along j
    assert _native._lm2exp_b_operand(b_t, 0) is b_t
    assert _native._lm2exp_b_operand(b_t, 1282) is b_t
    assert _native._lm2exp_b_operand(b_t, 2564) is not b_t      # pair tile: copy
    assert _native._lm2exp_b_operand(b_t, 201281) is not b_t    # fused max pass: copy
    b_odd = torch.zeros(2, 64, 97)
    assert _native._lm2exp_b_operand(b_odd, 0, flop=1e6) is b_odd          # small problem: in place
    assert _native._lm2exp_b_operand(b_odd, 0, flop=1e12) is not b_odd     # large problem: padded copy
    assert _native._lm2exp_b_operand(b_odd, 2564, flop=1e6) is not b_odd   # pair tile asked for: copy
    assert _native._lm2exp_b_operand(b_odd, 0, flop=1e6, want_colmax=True) is not b_odd
    assert _native._in_place_small(b_odd, 1e6, 0, False) and not _native._in_place_small(b_odd, 1e12, 0, False)
    assert not _native._in_place_small(b_odd.double(), 1e6, 0, False)


def test_automatic_plans_of_lm2exp():
    """What a call runs for the benchmark shapes and around the size rule of the optimistic stabilisers (the plan
    queries need no GPU: without one they assume 148 SMs)."""
    plan, launches = _native.LIB.triturus_b200_lm2exp_plan, _native.LIB.triturus_b200_lm2exp_launches
    assert plan(32, 1024, 1024, 1024, 0, 0) == 2567 and launches(32, 1024, 1024, 1024, 0, 0) == 2      # cfg2, TF32
    assert plan(32, 1024, 1024, 1024, 1, 0) == 402564 and launches(32, 1024, 1024, 1024, 1, 0) == 4    # cfg2, 3xTF32
    assert plan(128, 256, 256, 8192, 0, 0) == 2567                                                      # cfg3
    assert plan(4, 256, 256, 256, 0, 0) == 201281 and launches(4, 256, 256, 256, 0, 0) == 1             # cfg1
    assert plan(64, 256, 256, 256, 0, 0) // 100000 == 2      # two row blocks but under 2e10 FLOP: one fused launch
    assert plan(256, 128, 256, 8192, 0, 0) // 100000 == 3    # one row block, long launch: optimistic fused max pass
    assert plan(4, 1024, 1024, 1024, 0, 0) == 102566         # a chunk of the host pipeline: pre-pass + pair kernel
    assert plan(32, 1024, 1024, 1024, 0, 100000) == 102566   # forced pre-pass
    assert plan(32, 1024, 1024, 1024, 0, 2564) == 102564     # explicit tiles keep the exact stabiliser
    assert plan(32, 1024, 1024, 1024, 0, 402567) < 0 and plan(32, 1024, 1024, 1024, 1, 2567) < 0


def test_plans_over_random_shapes_are_consistent():
    """Invariants of the automatic plans over a few thousand random shapes (no GPU needed): the code decodes to a
    known tile and stabiliser, pins itself (asked for as an explicit variant it comes back unchanged), agrees with
    the launch count, and takes the optimistic forms only from 2e10 FLOP on."""
    import random

    rnd = random.Random(5)
    lm_plan, lm_launches = _native.LIB.triturus_b200_lm2exp_plan, _native.LIB.triturus_b200_lm2exp_launches
    lt_plan, lt_launches = _native.LIB.triturus_b200_lt2exp_plan, _native.LIB.triturus_b200_lt2exp_launches
    dims = [1, 3, 31, 32, 33, 64, 100, 127, 128, 129, 200, 256, 257, 384, 512, 1000, 1024, 2048, 4096, 8192]
    for _ in range(3000):
        R = rnd.choice([1, 2, 4, 7, 16, 32, 64, 128, 384])
        I, J, K = rnd.choice(dims), rnd.choice(dims), rnd.choice(dims)
        prec = rnd.choice([0, 1])
        code, n = lm_plan(R, I, J, K, prec, 0), lm_launches(R, I, J, K, prec, 0)
        assert code > 0, (R, I, J, K, prec, code)
        stab, tile = code // 100000, code % 100000
        assert tile in (1281, 1282, 2561, 2562, 2564, 2566, 2567), (R, I, J, K, prec, code)
        if tile in (2566, 2567):
            assert prec == 0 and I > 128, (R, I, J, K, code)
        if tile == 2567:
            assert stab == 0 and n == 2
        else:
            assert stab in (1, 2, 3, 4) and n == {1: 2, 2: 1, 3: 2, 4: 4}[stab], (R, I, J, K, prec, code, n)
        if tile == 2567 or stab in (3, 4):
            assert 2.0 * R * I * J * K >= 2e10, (R, I, J, K, prec, code)
        if stab == 4:
            assert tile == 2564
        if stab in (2, 3):
            assert tile in (1281, 1282, 2561, 2562)
        assert lm_plan(R, I, J, K, prec, code) == code, (R, I, J, K, prec, code)
        assert lm_launches(R, I, J, K, prec, code) == n

    for _ in range(3000):
        R = rnd.choice([1, 2, 4, 16, 64, 128])
        S = rnd.choice(dims[:-2])
        I, J = rnd.choice(dims[:14]), rnd.choice(dims[:14])
        K = rnd.choice(dims)
        prec = rnd.choice([0, 1])
        code, n = lt_plan(R, S, I, J, K, prec, 0), lt_launches(R, S, I, J, K, prec, 0)
        assert code > 0, (R, S, I, J, K, prec, code)
        split, tile = code // 10000, code % 10000
        assert tile in (1281, 1282, 2561, 2562, 1283, 1284, 1285), (R, S, I, J, K, prec, code)
        if tile in (1283, 1284, 1285):
            assert prec == 0
        assert split == 9998 or 1 <= split <= 4096, (R, S, I, J, K, prec, code)
        if split == 9998:  # shared last wave: in place (1 launch) or through zero-fill and log pass (3)
            assert n in (1, 3)
        else:
            assert n == (1 if split == 1 else 3), (R, S, I, J, K, prec, code, n)
        assert lt_plan(R, S, I, J, K, prec, code) == code, (R, S, I, J, K, prec, code)

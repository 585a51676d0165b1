"""GPU: this library against the reference's own Triton kernels, run on the same device and the same inputs.

Needs the unmodified reference under baseline/_ref (baseline/install_reference.py puts it there; the folder is
not part of this repository) and an importable Triton; otherwise every test here is skipped with the reason.

* `lm2exp` (triturus/lm2exp.py:167-206) and `lt2exp(..., mode="unsplit")` (triturus/lt2exp.py:519-630) are
  compared with this library's ops on the reference's test shapes (tests/lm2exp.py:13, tests/lt2exp.py:19)
  and on reduced copies of the five benchmark distributions, with the reference's TF32 flag off and on.
  The reference's `mode="split"` kernel is never launched: its merge is a spin lock without a bound
  (triturus/lt2exp.py:498-506).
* The reference's two hot-path test files are run unmodified, in a child pytest, with this repository's
  drop-in `triturus` package first on the path.
"""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from conftest import ATOL
from oracle import logspace_oracle as orc

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from baseline import reference_loader as rl  # noqa: E402

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(rl.available() is not None, reason=str(rl.available()))]


def _ref():
    try:
        return rl.load()
    except Exception as exc:  # noqa: BLE001  (e.g. a Triton that cannot initialise on this box)
        pytest.skip(f"the reference cannot be loaded: {exc}")


def _ref_call(fn, *args, **kw):
    """Run a reference kernel; a Triton compile failure on this architecture is a skip with the message."""
    try:
        out = fn(*args, **kw)
        torch.cuda.synchronize()
        return out
    except AssertionError:
        raise
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"the reference's Triton kernel did not run here: {type(exc).__name__}: {str(exc)[:300]}")


def _lm_cases():
    from triturus_b200.workloads import WORKLOADS

    yield "reftest", None, (24, 150, 100, 200)
    yield "cfg1", WORKLOADS["cfg1"], None
    yield "cfg2-R2", WORKLOADS["cfg2"].with_batch(2), None
    yield "cfg3-R4", WORKLOADS["cfg3"].with_batch(4), None


def _lt_cases():
    from triturus_b200.workloads import WORKLOADS, Workload

    yield "reftest", None, (3, 75, 50, 50, 100)
    yield "cfg4-R2", WORKLOADS["cfg4"].with_batch(2), None
    c5 = WORKLOADS["cfg5"]
    yield "cfg5-small", Workload("cfg5", "lt2exp", {**c5.dims, "R": 1, "S": 128, "K": 512}, c5.description), None


@pytest.mark.parametrize("allow_tf32", [False, True])
@pytest.mark.parametrize("case", list(_lm_cases()), ids=lambda c: c[0])
def test_lm2exp_against_reference_triton_kernel(case, allow_tf32):
    import triturus_b200 as tb
    from triturus_b200.workloads import make_inputs

    ref = _ref()
    name, wl, shape = case
    if wl is None:
        g = torch.Generator().manual_seed(42)
        R, I, J, K = shape
        a, b = torch.rand(R, I, J, generator=g), torch.randn(R, J, K, generator=g)
    else:
        a, b = make_inputs(wl, seed=0)
    ad, bd = a.cuda(), b.cuda()
    precision = "tf32" if allow_tf32 else "3xtf32"
    ref.set_tf32_enabled(allow_tf32)
    try:
        theirs = _ref_call(ref.lm2exp, ad, bd)
    finally:
        ref.set_tf32_enabled(False)
    ours = tb.lm2exp(ad, bd, precision=precision)
    tb.check_status()
    want = orc.lm2exp_fp64(a, b)
    res = orc.compare_logspace(ours.cpu(), want, ATOL[precision])
    assert res["ok"], res
    assert torch.equal(torch.isinf(theirs), torch.isinf(ours))
    fin = torch.isfinite(ours)
    diff = (theirs - ours)[fin].abs().max().item()
    # two implementations, each inside the stated tolerance of the float64 value
    assert diff <= 2 * ATOL[precision], diff
    if wl is None:
        # the reference's own acceptance bound (tests/lm2exp.py:20-23), Triton kernel in the role of ground truth
        assert torch.allclose(theirs, ours, rtol=5e-4 if allow_tf32 else 1e-5, atol=1e-6)


@pytest.mark.parametrize("allow_tf32", [False, True])
@pytest.mark.parametrize("case", list(_lt_cases()), ids=lambda c: c[0])
def test_lt2exp_against_reference_triton_kernel(case, allow_tf32):
    import triturus_b200 as tb
    from triturus_b200.workloads import make_inputs

    ref = _ref()
    name, wl, shape = case
    if wl is None:
        g = torch.Generator().manual_seed(42)
        R, S, I, J, K = shape
        w = torch.rand(R, S, I, J, generator=g)
        a, b = torch.randn(R, I, K, generator=g), torch.randn(R, J, K, generator=g)
    else:
        w, a, b = make_inputs(wl, seed=0)
    wd, ad, bd = w.cuda(), a.cuda(), b.cuda()
    precision = "tf32" if allow_tf32 else "3xtf32"
    ref.set_tf32_enabled(allow_tf32)
    try:
        theirs = _ref_call(ref.lt2exp, wd, ad, bd, mode="unsplit")
    finally:
        ref.set_tf32_enabled(False)
    for mode in ("unsplit", "auto"):
        ours = tb.lt2exp(wd, ad, bd, mode=mode, precision=precision)
        tb.check_status()
        want = orc.lt2exp_fp64(w, a, b)
        res = orc.compare_logspace(ours.cpu(), want, ATOL[precision])
        assert res["ok"], (mode, res)
        assert torch.equal(torch.isinf(theirs), torch.isinf(ours))
        fin = torch.isfinite(ours)
        diff = (theirs - ours)[fin].abs().max().item()
        assert diff <= 2 * ATOL[precision], (mode, diff)
        if wl is None:
            assert torch.allclose(theirs, ours, rtol=5e-4 if allow_tf32 else 1e-5, atol=1e-6)  # tests/lt2exp.py:37-40


def _child_pytest(pythonpath, extra):
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join(str(p) for p in pythonpath)
    env.pop("PYTEST_CURRENT_TEST", None)
    if os.path.exists("/usr/bin/g++"):
        env["CXX"] = "/usr/bin/g++"  # torch.compile's host-side code needs a g++ with OpenMP support
    suite = rl.SUITE_DIR
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider", "--rootdir", str(suite), "-c", os.devnull,
           str(suite / "tests" / "lm2exp.py"), str(suite / "tests" / "lt2exp.py"), *extra]  # fmt: skip
    return subprocess.run(cmd, cwd=str(suite), env=env, capture_output=True, text=True, timeout=1500)


def test_reference_test_files_pass_unmodified_on_the_drop_in_package():
    """tests/lm2exp.py and tests/lt2exp.py of the reference (8 items: both TF32 settings; modes auto, split and
    unsplit) with `triturus` resolving to this repository's package and `baselines` to the reference's."""
    if not (rl.SUITE_DIR / "tests" / "lm2exp.py").exists():
        pytest.skip("baseline/_ref/suite holds no copy of the reference's tests")
    proc = _child_pytest([ROOT, rl.SUITE_DIR], [])
    tail = (proc.stdout + proc.stderr)[-3000:]
    assert proc.returncode == 0, tail
    assert "8 passed" in proc.stdout, tail


def test_reference_passes_its_own_tests_here():
    """The same files against the reference's own Triton kernels on this GPU (the `split` items are deselected:
    unbounded spin lock).  Informational: a reference that cannot run here is a skip, with its output."""
    if not (rl.SUITE_DIR / "tests" / "lm2exp.py").exists():
        pytest.skip("baseline/_ref/suite holds no copy of the reference's tests")
    proc = _child_pytest([rl.REF_DIR, rl.SUITE_DIR], ["-k", "lm2exp or unsplit"])
    tail = (proc.stdout + proc.stderr)[-1500:]
    if proc.returncode != 0:
        pytest.skip(f"the reference's own suite did not pass on this box: {tail}")
    assert "4 passed" in proc.stdout, tail

"""CPU: pin the oracle against fixtures produced by the reference's own torch baselines."""

import pytest
import torch

from conftest import LM_GOLDEN, LT_GOLDEN, load_golden
from oracle import logspace_oracle as orc


def _same_inf(x, y):
    return torch.equal(torch.isinf(x), torch.isinf(y)) and torch.equal(x[torch.isinf(x)], y[torch.isinf(y)])


@pytest.mark.parametrize("name", LM_GOLDEN)
def test_lm2exp_fp32_matches_reference_baseline(name):
    g = load_golden(name)
    got = orc.lm2exp_fp32(g["a"], g["b"])
    assert not torch.isnan(got).any()
    assert _same_inf(got, g["out"])
    fin = torch.isfinite(g["out"])
    # same formula, same fp32 ops: only bmm's summation order may differ
    assert torch.allclose(got[fin], g["out"][fin], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", LM_GOLDEN)
def test_lm2exp_fp64_brackets_reference_baseline(name):
    g = load_golden(name)
    res = orc.compare_logspace(g["out"], orc.lm2exp_fp64(g["a"], g["b"]), atol=5e-5)
    assert res["ok"], res


@pytest.mark.parametrize("name", LT_GOLDEN)
def test_lt2exp_fp32_matches_reference_baseline(name):
    g = load_golden(name)
    got = orc.lt2exp_fp32(g["w"], g["a"], g["b"])
    assert not torch.isnan(got).any()
    assert _same_inf(got, g["out"])
    fin = torch.isfinite(g["out"])
    assert torch.allclose(got[fin], g["out"][fin], rtol=1e-5, atol=1e-6)
    assert torch.allclose(got[fin], g["out_einsum"][fin], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", LT_GOLDEN)
def test_lt2exp_fp64_brackets_reference_baseline(name):
    g = load_golden(name)
    want = orc.lt2exp_fp64(g["w"], g["a"], g["b"], chunk=2)
    res = orc.compare_logspace(g["out"], want, atol=5e-5)
    assert res["ok"], res


def test_all_neginf_column_gives_neginf_not_nan():
    a = torch.rand(1, 4, 6)
    b = torch.randn(1, 6, 5)
    b[0, :, 2] = float("-inf")
    out = orc.lm2exp_fp32(a, b)
    assert torch.all(out[0, :, 2] == float("-inf"))
    assert not torch.isnan(out).any()
    w = torch.rand(1, 3, 4, 6)
    x = torch.randn(1, 4, 5)
    x[0, :, 1] = float("-inf")
    out = orc.lt2exp_fp32(w, x, b)
    assert torch.all(out[0, :, 1] == float("-inf")) and torch.all(out[0, :, 2] == float("-inf"))
    assert not torch.isnan(out).any()


def test_fp64_chunking_is_exact():
    g = load_golden("lt_cfg4")
    a1 = orc.lt2exp_fp64(g["w"], g["a"], g["b"], chunk=1)
    a2 = orc.lt2exp_fp64(g["w"], g["a"], g["b"], chunk=2)
    assert torch.equal(a1, a2)


def test_compare_logspace_flags_problems():
    want = torch.tensor([0.0, float("-inf"), 1.0])
    assert orc.compare_logspace(want.clone(), want, 1e-6)["ok"]
    assert not orc.compare_logspace(torch.tensor([0.0, -1e30, 1.0]), want, 1e-6)["ok"]
    assert not orc.compare_logspace(torch.tensor([0.0, float("-inf"), float("nan")]), want, 1e-6)["ok"]
    assert not orc.compare_logspace(torch.tensor([0.1, float("-inf"), 1.0]), want, 1e-6)["ok"]


def test_oracle_rejects_bad_shapes():
    with pytest.raises(ValueError):
        orc.lm2exp_fp32(torch.rand(2, 3, 4), torch.rand(2, 5, 6))
    with pytest.raises(ValueError):
        orc.lt2exp_fp32(torch.rand(2, 3, 4, 5), torch.rand(2, 4, 6), torch.rand(2, 4, 6))

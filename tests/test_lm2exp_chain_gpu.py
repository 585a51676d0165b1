"""GPU tests of lm2exp used as a link of a chain of layers: the epilogue's column maxima of the result
(`return_colmax`) and a caller-supplied stabiliser (`b_colmax`).  The chained results must equal the
unchained ones within the same log-space tolerances vs float64 (2e-3 TF32, 1e-4 3xTF32), the returned maxima
must be exactly the maxima of the values written, and -inf columns must stay -inf through the chain."""

import ctypes

import pytest
import torch

from conftest import ATOL
from oracle import logspace_oracle as orc

pytestmark = pytest.mark.gpu

PRECISIONS = ["tf32", "3xtf32"]


def _inputs(R, I, J, K, seed, scale=5.0):
    g = torch.Generator().manual_seed(seed)
    a = torch.rand(R, I, J, generator=g) + 0.01
    b = torch.randn(R, J, K, generator=g) * scale + 50.0 * torch.randn(R, 1, K, generator=g)
    return a, b


def _lm2exp_all_fp64(a64, b64):
    """The oracle's float64 formula (oracle/logspace_oracle.py, lm2exp_fp64) on float64 inputs, so that a
    chain of layers is evaluated without rounding the intermediate results to float32."""
    m = b64.amax(dim=1, keepdim=True).clamp(min=-1e300, max=1e300)
    return torch.bmm(a64, (b64 - m).exp()).log() + m


# (shape, variant): single-CTA tiles with one and several row tiles, the CTA-pair kernel, ragged edges.
CASES = [
    ((2, 100, 70, 130), 0),
    ((3, 300, 171, 530), 1281),
    ((3, 300, 171, 530), 1282),
    ((3, 300, 171, 530), 2561),
    ((2, 520, 96, 515), 2564),
    ((1, 1024, 256, 1024), 0),
    ((1, 7, 5, 3), 0),
]


@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("shape,variant", CASES)
def test_returned_colmax_is_the_maximum_of_the_result(shape, variant, precision):
    import triturus_b200 as tb

    a, b = _inputs(*shape, seed=sum(shape))
    out, m = tb.lm2exp(a.cuda(), b.cuda(), precision=precision, variant=variant, return_colmax=True)
    plain = tb.lm2exp(a.cuda(), b.cuda(), precision=precision, variant=variant)
    tb.check_status()
    assert m.shape == (shape[0], shape[3])
    assert torch.equal(out, plain)                      # emitting the maxima does not change the result
    assert torch.equal(m, out.amax(dim=1))              # bit-exact: a maximum of stored values
    res = orc.compare_logspace(out.cpu(), orc.lm2exp_fp64(a, b), ATOL[precision])
    assert res["ok"], res


@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("shape,variant", CASES)
def test_supplied_colmax_replaces_the_stabiliser_pass(shape, variant, precision):
    import triturus_b200 as tb

    a, b = _inputs(*shape, seed=17 + sum(shape))
    bd = b.cuda()
    m = bd.amax(dim=1)                                  # unclamped: the kernel clamps on read
    got = tb.lm2exp(a.cuda(), bd, precision=precision, variant=variant, b_colmax=m)
    tb.check_status()
    res = orc.compare_logspace(got.cpu(), orc.lm2exp_fp64(a, b), ATOL[precision])
    assert res["ok"], res
    # same stabiliser values as the library's own pre-pass
    assert torch.equal(tb.colmax(bd), m.clamp(-1e38, 1e38))


@pytest.mark.parametrize("precision", PRECISIONS)
def test_three_layer_chain_matches_unchained_and_float64(precision):
    import triturus_b200 as tb

    R, K = 4, 700
    dims = [260, 384, 130, 513]                         # layer n maps dims[n] -> dims[n + 1] rows
    g = torch.Generator().manual_seed(5)
    x0 = torch.randn(R, dims[0], K, generator=g) * 6.0 - 30.0 * torch.rand(R, 1, K, generator=g)
    x0[0, :, 11] = float("-inf")                        # a column that stays -inf through every layer
    x0[torch.rand(x0.shape, generator=g) < 0.02] = float("-inf")
    ws = [torch.softmax(torch.randn(R, dims[n + 1], dims[n], generator=g), dim=-1) for n in range(3)]

    x_chain, m = x0.cuda(), None
    x_plain = x0.cuda()
    x64 = x0.double()
    for w in ws:
        wd = w.cuda()
        x_chain, m = tb.lm2exp(wd, x_chain, precision=precision, b_colmax=m, return_colmax=True)
        x_plain = tb.lm2exp(wd, x_plain, precision=precision)
        x64 = _lm2exp_all_fp64(w.double(), x64)
    tb.check_status()
    assert not torch.isnan(x_chain).any()
    assert torch.all(x_chain[0, :, 11] == float("-inf")) and torch.all(m[0, 11] == float("-inf"))
    # three layers accumulate three layers' worth of rounding
    res = orc.compare_logspace(x_chain.cpu(), x64, 3 * ATOL[precision])
    assert res["ok"], res
    res = orc.compare_logspace(x_chain.cpu(), x_plain.cpu().double(), 3 * ATOL[precision])
    assert res["ok"], res
    assert torch.equal(m, x_chain.amax(dim=1))


def test_chain_launch_counts_and_c_abi_argument_checks():
    import triturus_b200 as tb
    from triturus_b200 import _native

    lib = _native.LIB
    # cfg2 shape: pre-pass + contraction; with a supplied stabiliser one launch; + 1 fill for the maxima
    assert lib.triturus_b200_lm2exp_chain_launches(32, 1024, 1024, 1024, 0, 0, 0, 0) == 2  # optimistic stabiliser + its conditional launch
    assert lib.triturus_b200_lm2exp_chain_launches(32, 1024, 1024, 1024, 1, 0, 0, 0) == 4  # 3xTF32: 32-row pre-pass
    assert lib.triturus_b200_lm2exp_chain_launches(32, 1024, 1024, 1024, 1, 100000, 0, 0) == 2
    assert lib.triturus_b200_lm2exp_chain_launches(32, 1024, 1024, 1024, 0, 0, 1, 0) == 1
    assert lib.triturus_b200_lm2exp_chain_launches(32, 1024, 1024, 1024, 0, 0, 1, 1) == 2
    assert lib.triturus_b200_lm2exp_chain_launches(32, 1024, 1024, 1024, 0, 202561, 1, 0) < 0

    a, b = _inputs(2, 64, 32, 64, seed=1)
    ad, bd = a.cuda(), b.cuda()
    out = torch.empty(2, 64, 64, device="cuda")
    m = bd.amax(dim=1).contiguous()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    i64 = ctypes.c_int64 * 3
    args = (ad.data_ptr(), bd.data_ptr(), out.data_ptr(), 2, 64, 32, 64, i64(*ad.stride()), i64(*bd.stride()),
            i64(*out.stride()), 0)
    stream = torch.cuda.current_stream().cuda_stream
    # no workspace and no stabiliser: refused; same buffer for both maxima: refused; a fused max pass
    # requested together with a supplied stabiliser: refused
    assert lib.triturus_b200_lm2exp_chain_f32(*args, 0, None, None, None, 0, st.data_ptr(), stream) != 0
    assert lib.triturus_b200_lm2exp_chain_f32(*args, 0, m.data_ptr(), m.data_ptr(), None, 0, st.data_ptr(), stream) != 0
    assert lib.triturus_b200_lm2exp_chain_f32(*args, 201281, m.data_ptr(), None, None, 0, st.data_ptr(), stream) != 0
    # with the stabiliser supplied, no workspace is needed
    assert lib.triturus_b200_lm2exp_chain_f32(*args, 0, m.data_ptr(), None, None, 0, st.data_ptr(), stream) == 0
    tb.check_status()
    res = orc.compare_logspace(out.cpu(), orc.lm2exp_fp64(a, b), ATOL["tf32"])
    assert res["ok"], res

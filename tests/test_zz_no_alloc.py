"""GPU: the lm2exp entry point for callers that may not allocate device memory.

Such callers (arena-owned HBM, allocation-free serving loops, plugin hosts that receive only input and
output buffers) use `triturus_b200_lm2exp_f32_static`, whose stabiliser scratch is a fixed array inside
the library.  This test drives it through the C ABI with ctypes, twice in a row with different problem
sizes.  Both calls are pinned to the kernels that take their stabiliser from the scratch array (the
pre-pass writes it, the contraction kernel reads it), so the second call really finds the first call's
leftovers there.  Each result is checked against the float64 CPU oracle and, bit for bit, against the
entry point that takes a caller workspace.  It also checks that oversize problems are refused.

The file name sorts last on purpose: a failure here cannot hide the rest of the suite under `-x`.
"""

import ctypes

import pytest
import torch

from conftest import ATOL
from oracle import logspace_oracle as orc

pytestmark = pytest.mark.gpu


PREPASS = 100000  # variant code: stabiliser from the pre-pass through the scratch array, never the fused max pass


def _call_static(a, b, precision):
    from triturus_b200 import _native

    R, I, J = a.shape
    K = b.shape[2]
    out = torch.empty((R, I, K), dtype=torch.float32, device=a.device)
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    stream = torch.cuda.current_stream(a.device).cuda_stream
    rc = _native.LIB.triturus_b200_lm2exp_f32_static(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), R, I, J, K,
        _native._i64(a.stride()), _native._i64(b.stride()), _native._i64(out.stride()),
        precision, PREPASS, status.data_ptr(), stream,
    )  # fmt: skip
    assert rc == 0, _native.strerror(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out


@pytest.mark.parametrize("precision", [0, 1])
def test_static_scratch_entry_matches_oracle_twice(precision):
    from triturus_b200 import _native

    name = "tf32" if precision == 0 else "3xtf32"
    g = torch.Generator().manual_seed(31)
    # first call fills a large part of the built-in array, second call is smaller and has other maxima
    shapes = [(8, 300, 160, 4096), (3, 130, 96, 520)]
    for R, I, J, K in shapes:
        # both calls launch the pre-pass and the contraction kernel (two launches): the array is written and read
        assert _native.LIB.triturus_b200_lm2exp_launches(R, I, J, K, precision, PREPASS) == 2
        a = torch.rand(R, I, J, generator=g)
        b = torch.randn(R, J, K, generator=g) * 6.0 + 80.0 * torch.randn(R, 1, K, generator=g)
        b[0, :, 3] = float("-inf")
        got = _call_static(a.cuda(), b.cuda(), precision)
        res = orc.compare_logspace(got.cpu(), orc.lm2exp_fp64(a, b), ATOL[name])
        assert res["ok"], res
        assert torch.all(got[0, :, 3] == float("-inf"))
        # same kernels, same stabiliser values, other scratch memory: identical bits
        same = _native._lm2exp_impl(a.cuda(), b.cuda(), precision, PREPASS)
        torch.cuda.synchronize()
        assert torch.equal(got, same)


def test_static_scratch_entry_rejects_oversize_problems():
    from triturus_b200 import _native

    lib = _native.LIB
    limit = int(lib.triturus_b200_lm2exp_static_max_columns())
    assert limit == 1 << 20
    a = torch.rand(1, 8, 8).cuda()
    s3 = _native._i64([64, 8, 1])
    # R * K just over the limit: refused before anything is launched, whatever the pointers are
    rc = lib.triturus_b200_lm2exp_f32_static(
        a.data_ptr(), a.data_ptr(), a.data_ptr(), 2, 8, 8, limit // 2 + 1, s3, s3, s3, 0, 0, None, None
    )
    assert rc == -7 and "static" in _native.strerror(rc)
    torch.cuda.synchronize()

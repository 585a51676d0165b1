"""GPU: the bounded-wait error path that every kernel of the library shares, made to run once.

No input can make a real kernel's wait run out, so the library carries a self-test launch
(`triturus_b200_selftest_wait_timeout`): one warp waits on a barrier that nobody signals, with a wait limit of
a few hundred microseconds instead of the kernels' ~1.5 s.  The wait gives up, the kernel returns by itself with
an error code in the status word, and the host side turns that code into `NativeLibraryError`.  Nothing traps,
faults or spins without a bound, and the CUDA context stays usable, which the test checks with a real call
afterwards.
"""

import pytest
import torch

from conftest import ATOL
from oracle import logspace_oracle as orc

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_is_reported_and_the_context_survives():
    import triturus_b200 as tb
    from triturus_b200 import _native

    dev = torch.device("cuda", 0)
    tb.check_status(dev)  # clean slate
    status = _native._status_word(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    rc = _native.LIB.triturus_b200_selftest_wait_timeout(status.data_ptr(), 400_000, stream)  # ~0.2 ms
    assert rc == 0, _native.strerror(rc)
    with pytest.raises(tb.NativeLibraryError, match="105.*setup wait timed out"):
        tb.check_status(dev)
    # the status word was cleared by the failed check and the context still works
    tb.check_status(dev)
    g = torch.Generator().manual_seed(3)
    a, b = torch.rand(2, 70, 50, generator=g), torch.randn(2, 50, 90, generator=g)
    out = tb.lm2exp(a.cuda(), b.cuda(), precision="3xtf32")
    tb.check_status(dev)
    res = orc.compare_logspace(out.cpu(), orc.lm2exp_fp64(a, b), ATOL["3xtf32"])
    assert res["ok"], res


def test_selftest_refuses_long_or_missing_arguments():
    from triturus_b200 import _native

    status = _native._status_word(torch.device("cuda", 0))
    lib = _native.LIB
    assert lib.triturus_b200_selftest_wait_timeout(None, 400_000, None) == -1
    assert lib.triturus_b200_selftest_wait_timeout(status.data_ptr(), 10**12, None) == -1  # no long spins on request
    assert lib.triturus_b200_selftest_wait_timeout(status.data_ptr(), 10, None) == -1

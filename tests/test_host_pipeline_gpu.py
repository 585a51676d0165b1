"""The pipelined host-tensor entry points (triturus_b200/host.py) against the device entry points and the
float64 oracle: chunked batches, caller-supplied pinned output, pageable inputs."""

import pytest
import torch

from conftest import ATOL
from oracle import logspace_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chunks", [None, 1, 3, 16])
def test_lm2exp_host_matches_device_call(chunks):
    import triturus_b200 as tb

    g = torch.Generator().manual_seed(31)
    a = torch.rand(7, 150, 90, generator=g).pin_memory()
    b = (torch.randn(7, 90, 200, generator=g) * 5.0).pin_memory()
    b[3, :, 17] = float("-inf")
    out = tb.lm2exp_host(a, b, chunks=chunks, precision="3xtf32", variant=1281)
    torch.cuda.current_stream().synchronize()
    assert out.shape == (7, 150, 200) and out.is_pinned() and not out.is_cuda
    direct = tb.lm2exp(a.cuda(), b.cuda(), precision="3xtf32", variant=1281).cpu()
    tb.check_status()
    assert torch.equal(out, direct)
    res = orc.compare_logspace(out, orc.lm2exp_fp64(a, b), ATOL["3xtf32"])
    assert res["ok"], res


@pytest.mark.parametrize("chunks", [None, 2, 5])
def test_lt2exp_host_matches_device_call(chunks):
    import triturus_b200 as tb

    g = torch.Generator().manual_seed(32)
    w = torch.rand(5, 130, 9, 33, generator=g)   # pageable on purpose
    a = torch.randn(5, 9, 140, generator=g) * 3.0
    b = torch.randn(5, 33, 140, generator=g) * 3.0
    out_buf = torch.full((5, 130, 140), 9.0).pin_memory()
    out = tb.lt2exp_host(w, a, b, out=out_buf, chunks=chunks, mode="unsplit", precision="tf32", variant=1281)
    torch.cuda.current_stream().synchronize()
    assert out is out_buf
    direct = tb.lt2exp(w.cuda(), a.cuda(), b.cuda(), mode="unsplit", precision="tf32", variant=1281).cpu()
    tb.check_status()
    assert torch.equal(out, direct)
    res = orc.compare_logspace(out, orc.lt2exp_fp64(w, a, b), ATOL["tf32"])
    assert res["ok"], res


def test_host_entry_points_order_after_the_current_stream():
    """Work queued on the current stream after the call sees the finished result without a host sync."""
    import triturus_b200 as tb

    g = torch.Generator().manual_seed(33)
    a = torch.rand(8, 256, 256, generator=g).pin_memory()
    b = torch.randn(8, 256, 256, generator=g).pin_memory()
    out = tb.lm2exp_host(a, b, chunks=4, precision="tf32")
    back = out.to("cuda", non_blocking=True)   # ordered on the current stream
    want = tb.lm2exp(a.cuda(), b.cuda(), precision="tf32")
    torch.cuda.synchronize()
    assert (back - want).abs().max().item() <= 2 * ATOL["tf32"]
    tb.check_status()


def test_host_entry_points_refuse_cuda_and_bad_out():
    import triturus_b200 as tb

    a = torch.rand(2, 8, 8)
    b = torch.rand(2, 8, 8)
    with pytest.raises(ValueError):
        tb.lm2exp_host(a.cuda(), b.cuda())
    with pytest.raises(ValueError):
        tb.lm2exp_host(a, b, out=torch.empty(2, 8, 9))

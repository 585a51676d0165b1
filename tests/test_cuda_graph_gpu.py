"""Both ops under CUDA-graph capture: the entry points neither synchronise nor allocate on their own, so a
captured call can be replayed on new input values (launch-bound inner loops of a caller)."""

import pytest
import torch

from conftest import ATOL
from oracle import logspace_oracle as orc

pytestmark = pytest.mark.gpu


def _capture(fn, *static_inputs):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn(*static_inputs)  # warm-up outside the capture (lazy attribute set-up, allocator pool)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            out = fn(*static_inputs)
    torch.cuda.current_stream().wait_stream(s)
    return graph, out


@pytest.mark.parametrize("variant", [0, 101281, 2564])
def test_lm2exp_graph_replay(variant):
    import triturus_b200 as tb

    g = torch.Generator().manual_seed(41)
    I = 600 if variant == 2564 else 96
    a = torch.rand(2, I, 200, generator=g).cuda()
    b = torch.randn(2, 200, 300, generator=g).cuda()
    graph, out = _capture(lambda x, y: tb.lm2exp(x, y, precision="tf32", variant=variant), a, b)
    for seed in (1, 2):
        g2 = torch.Generator().manual_seed(seed)
        a.copy_(torch.rand(2, I, 200, generator=g2))
        b.copy_(torch.randn(2, 200, 300, generator=g2) * 3.0)
        graph.replay()
        torch.cuda.synchronize()
        res = orc.compare_logspace(out.cpu(), orc.lm2exp_fp64(a.cpu(), b.cpu()), ATOL["tf32"])
        assert res["ok"], res
    tb.check_status()


@pytest.mark.parametrize("variant,precision", [(2567, "tf32"), (402564, "3xtf32"), (301282, "tf32")])
def test_optimistic_stabilisers_under_graph_replay(variant, precision):
    """The optimistic forms captured once (the contraction, the flag hand-over and the conditional launches of the
    exact passes, chained as programmatic dependents) and replayed on inputs that keep the optimistic result, then
    on inputs that overflow it, then on benign ones again: the flag words live in the workspace the capture holds,
    are raised and put down by the captured kernels themselves, and every replay is right."""
    import triturus_b200 as tb

    g = torch.Generator().manual_seed(43)
    R, I, J, K = 2, 512, 256, 300
    a = torch.rand(R, I, J, generator=g).cuda()
    b = torch.randn(R, J, K, generator=g).cuda()
    graph, out = _capture(lambda x, y: tb.lm2exp(x, y, precision=precision, variant=variant), a, b)
    ramp = torch.arange(J, dtype=torch.float32).view(1, J, 1) * 2.0  # rows far above the first 32: overflow
    for step, kind in enumerate(("benign", "overflow", "benign", "overflow", "benign")):
        g2 = torch.Generator().manual_seed(100 + step)
        bb = torch.randn(R, J, K, generator=g2) * 3.0
        if kind == "overflow":
            bb = bb + ramp
        a.copy_(torch.rand(R, I, J, generator=g2))
        b.copy_(bb)
        graph.replay()
        torch.cuda.synchronize()
        res = orc.compare_logspace(out.cpu(), orc.lm2exp_fp64(a.cpu(), b.cpu()), ATOL[precision])
        assert res["ok"], (kind, step, res)
    tb.check_status()


@pytest.mark.parametrize("mode", ["unsplit", "split"])
def test_lt2exp_graph_replay(mode):
    """The split mode captures three kernels (zero-fill, slices, log pass)."""
    import triturus_b200 as tb

    g = torch.Generator().manual_seed(42)
    w = torch.rand(1, 100, 24, 40, generator=g).cuda()
    a = torch.randn(1, 24, 130, generator=g).cuda()
    b = torch.randn(1, 40, 130, generator=g).cuda()
    graph, out = _capture(lambda x, y, z: tb.lt2exp(x, y, z, mode=mode, precision="3xtf32"), w, a, b)
    for seed in (3, 4):
        g2 = torch.Generator().manual_seed(seed)
        w.copy_(torch.rand(1, 100, 24, 40, generator=g2))
        a.copy_(torch.randn(1, 24, 130, generator=g2) * 2.0)
        graph.replay()
        torch.cuda.synchronize()
        res = orc.compare_logspace(out.cpu(), orc.lt2exp_fp64(w.cpu(), a.cpu(), b.cpu()), ATOL["3xtf32"])
        assert res["ok"], res
    tb.check_status()

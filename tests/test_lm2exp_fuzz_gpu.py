"""GPU: random shapes against the float64 oracle.

* through the optimistic stabilisers of lm2exp (variants 2567, 3xxxxx, 402564): every fourth case overflows the
  optimistic result after the first k-block (the conditional exact launch must take over), every fourth has -inf
  entries, every fourth nothing finite in its first 32 rows;
* with operands given as random views (transposed, strided, shifted by one element, broadcast over the batch),
  which the library reads in place: through tensor maps where the view allows it, element by element otherwise."""

import random

import pytest
import torch

from conftest import ATOL
from oracle import logspace_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [7, 8])
def test_random_shapes_through_the_optimistic_stabilisers(seed):
    import triturus_b200 as tb

    rnd = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    failures = []
    for trial in range(24):
        R = rnd.choice([1, 2, 3, 5])
        I, J, K = rnd.randint(1, 700), rnd.randint(1, 400), rnd.randint(1, 700)
        a = torch.rand(R, I, J, generator=g)
        b = torch.randn(R, J, K, generator=g) * rnd.choice([1.0, 5.0, 30.0]) + 40.0 * torch.randn(R, 1, K, generator=g)
        kind = trial % 4
        if kind == 1 and J > 40:
            b[:, 33:] += 200.0
        if kind == 2:
            b[torch.rand(R, J, K, generator=g) < 0.05] = float("-inf")
        if kind == 3 and J > 33:
            b[:, :32] = float("-inf")
        want = orc.lm2exp_fp64(a, b)
        ad, bd = a.cuda(), b.cuda()
        for precision, variants in (("tf32", (2567, 300000, 402564)), ("3xtf32", (300000, 402564))):
            for variant in variants:
                got = tb.lm2exp(ad, bd, precision=precision, variant=variant)
                tb.check_status()
                res = orc.compare_logspace(got.cpu(), want, ATOL[precision])
                if not res["ok"]:
                    failures.append(((R, I, J, K), precision, variant, kind, res))
    assert not failures, failures[:3]


def _random_view(rnd, g, shape):
    """A [R, X, Y] tensor with random values, stored in one of several layouts; returns (view on the GPU, dense CPU copy)."""
    R, X, Y = shape
    kind = rnd.choice(["plain", "transposed", "strided", "shifted", "broadcast", "padded"])
    if kind == "plain":
        v = torch.randn(R, X, Y, generator=g).cuda()
    elif kind == "transposed":
        v = torch.randn(R, Y, X, generator=g).cuda().transpose(1, 2)
    elif kind == "strided":
        v = torch.randn(R, X, 2 * Y + 1, generator=g).cuda()[:, :, 1::2][:, :, :Y]
    elif kind == "shifted":
        v = torch.randn(R * X * Y + 1, generator=g).cuda()[1:].view(R, X, Y)
    elif kind == "broadcast":
        v = torch.randn(1, X, Y, generator=g).cuda().expand(R, X, Y)
    else:
        v = torch.randn(R, X, Y + 3, generator=g).cuda()[:, :, :Y]
    return kind, v, v.cpu().contiguous()


@pytest.mark.parametrize("seed", [11, 12])
def test_random_views_are_read_without_error(seed):
    import triturus_b200 as tb

    rnd = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    failures = []
    for trial in range(20):
        R = rnd.choice([1, 2, 3])
        I, J, K = rnd.randint(1, 400), rnd.randint(1, 300), rnd.randint(1, 400)
        ka, av, a = _random_view(rnd, g, (R, I, J))
        kb, bv, b = _random_view(rnd, g, (R, J, K))
        av, a = av.abs(), a.abs()
        bv, b = bv * 4.0, b * 4.0
        want = orc.lm2exp_fp64(a, b)
        for precision in ("tf32", "3xtf32"):
            got = tb.lm2exp(av, bv, precision=precision)
            tb.check_status()
            res = orc.compare_logspace(got.cpu(), want, ATOL[precision])
            if not res["ok"]:
                failures.append(((R, I, J, K), ka, kb, precision, res))
    assert not failures, failures[:3]

"""GPU: random shapes through the optimistic stabilisers of lm2exp (variants 2567, 3xxxxx, 402564), against the
float64 oracle.  Every fourth case overflows the optimistic result after the first k-block (the conditional exact
launch must take over), every fourth has -inf entries, every fourth nothing finite in its first 32 rows."""

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

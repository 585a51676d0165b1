"""GPU: lt2exp on random shapes with a and b given as random views (transposed, strided, shifted by one element,
broadcast over the batch), all three modes, against the float64 oracle."""

import random

import pytest
import torch

from conftest import ATOL
from oracle import logspace_oracle as orc
from test_lm2exp_fuzz_gpu import _random_view

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [21, 22])
def test_random_shapes_and_views(seed):
    import triturus_b200 as tb

    rnd = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    failures = []
    for trial in range(16):
        R = rnd.choice([1, 2, 3])
        S, I, J, K = rnd.randint(1, 300), rnd.randint(1, 40), rnd.randint(1, 70), rnd.randint(1, 400)
        w = torch.rand(R, S, I, J, generator=g)
        ka, av, a = _random_view(rnd, g, (R, I, K))
        kb, bv, b = _random_view(rnd, g, (R, J, K))
        av, a, bv, b = av * 3.0, a * 3.0, bv * 3.0, b * 3.0
        want = orc.lt2exp_fp64(w, a, b)
        for precision in ("tf32", "3xtf32"):
            for mode in ("auto", "unsplit", "split"):
                got = tb.lt2exp(w.cuda(), av, bv, mode=mode, precision=precision)
                tb.check_status()
                res = orc.compare_logspace(got.cpu(), want, ATOL[precision])
                if not res["ok"]:
                    failures.append(((R, S, I, J, K), ka, kb, precision, mode, res))
    assert not failures, failures[:3]

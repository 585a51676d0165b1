"""Generate the golden fixtures in this directory by running the REFERENCE's own torch baselines.

Run in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports `baselines.lm2exp.lm2exp` and `baselines.lt2exp.lt2exp` / `lt2exp_einsum` from that checkout
(baselines/lm2exp.py:4, baselines/lt2exp.py:4,28), evaluates them on CPU on small seeded inputs, and stores
inputs and outputs as .npz files.  The cases cover the shapes of the reference's own tests
(tests/lm2exp.py:13, tests/lt2exp.py:19), scaled-down versions of the five benchmark distributions, and
the -inf edge cases.  The fixtures travel with the repository; the reference does not.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from triturus_b200.workloads import WORKLOADS, Workload, make_inputs  # noqa: E402


def small(name: str, **dims) -> Workload:
    wl = WORKLOADS[name]
    return Workload(wl.name, wl.op, {**wl.dims, **dims}, wl.description)


def lm_cases():
    g = torch.Generator().manual_seed(42)
    cases = {}
    # the reference's own test shape (tests/lm2exp.py:13-15) at batch 4 instead of 24 to keep the file small
    cases["lm_reftest"] = (torch.rand(4, 150, 100, generator=g), torch.randn(4, 100, 200, generator=g))
    cases["lm_cfg1"] = make_inputs(small("cfg1", R=2, I=64, J=96, K=80), seed=0)
    cases["lm_cfg2"] = make_inputs(small("cfg2", R=2, I=96, J=128, K=72), seed=0)
    cases["lm_cfg3"] = make_inputs(small("cfg3", R=3, I=40, J=64, K=260), seed=0)
    # edge: a whole column of b at -inf, isolated -inf, a row of zeros in a
    a = torch.rand(2, 33, 45, generator=g)
    b = torch.randn(2, 45, 37, generator=g) * 30.0
    b[0, :, 5] = float("-inf")
    b[1, :, 0] = float("-inf")
    b[0, 7, 9] = float("-inf")
    b[1, 44, 36] = float("-inf")
    a[1, 4, :] = 0.0
    cases["lm_neginf"] = (a, b)
    cases["lm_single"] = (torch.rand(1, 1, 1, generator=g), torch.randn(1, 1, 1, generator=g))
    return cases


def lt_cases():
    g = torch.Generator().manual_seed(42)
    cases = {}
    # the reference's own test shape (tests/lt2exp.py:19-22) at batch 1 instead of 3 to keep the file small
    cases["lt_reftest"] = (
        torch.rand(1, 75, 50, 50, generator=g),
        torch.randn(1, 50, 100, generator=g),
        torch.randn(1, 50, 100, generator=g),
    )
    cases["lt_cfg4"] = make_inputs(small("cfg4", R=2, S=40, I=12, J=20, K=72), seed=0)
    cases["lt_cfg5"] = make_inputs(small("cfg5", R=2, S=48, I=16, J=36, K=68), seed=0)
    w = torch.rand(2, 9, 7, 11, generator=g)
    a = torch.randn(2, 7, 21, generator=g) * 20.0
    b = torch.randn(2, 11, 21, generator=g) * 20.0
    a[0, :, 3] = float("-inf")
    b[1, :, 20] = float("-inf")
    a[1, 2, 5] = float("-inf")
    b[0, 10, 0] = float("-inf")
    cases["lt_neginf"] = (w, a, b)
    return cases


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from baselines.lm2exp import lm2exp as ref_lm2exp
    from baselines.lt2exp import lt2exp as ref_lt2exp
    from baselines.lt2exp import lt2exp_einsum as ref_lt2exp_einsum

    torch.set_num_threads(1)  # fixed summation order inside bmm
    for name, (a, b) in lm_cases().items():
        out = ref_lm2exp(a, b)
        np.savez_compressed(HERE / f"{name}.npz", a=a.numpy(), b=b.numpy(), out=out.numpy())
        print(name, tuple(out.shape), "-inf:", int((out == float("-inf")).sum()), "nan:", int(out.isnan().sum()))
    for name, (w, a, b) in lt_cases().items():
        out = ref_lt2exp(w, a, b)
        out_e = ref_lt2exp_einsum(w, a, b)
        np.savez_compressed(
            HERE / f"{name}.npz", w=w.numpy(), a=a.numpy(), b=b.numpy(), out=out.numpy(), out_einsum=out_e.numpy()
        )
        print(name, tuple(out.shape), "-inf:", int((out == float("-inf")).sum()), "nan:", int(out.isnan().sum()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of loreloc/triturus>")
    main(sys.argv[1])

"""The reference's benchmark sweeps for the hot path, as data.

Shapes and input distributions of `benchmarks/lm2exp.py:26-56,80-83` and `benchmarks/lt2exp.py:32-63,70-74`
(square and rectangular families, each with the TF32 flag off and on), and the reference's throughput
convention: GB/s over the INPUT elements only (`benchmarks/lm2exp.py:95`, `benchmarks/lt2exp.py:90`,
`benchmarks/utils.py:8-9`).  `bench.py --sweep` walks these families; `tests/test_sweep_shapes_gpu.py` checks
the results on them.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class SweepPoint:
    op: str        # "lm2exp" or "lt2exp"
    family: str    # the reference's plot name without the flag
    dims: dict     # reference letters: batch, m, k, n (lm2exp) / batch, m, j, k, n (lt2exp)

    @property
    def input_elems(self) -> int:
        d = self.dims
        if self.op == "lm2exp":
            return d["batch"] * (d["m"] * d["k"] + d["k"] * d["n"])
        return d["batch"] * (d["m"] * d["j"] * d["k"] + d["j"] * d["n"] + d["k"] * d["n"])

    @property
    def flops(self) -> float:
        d = self.dims
        if self.op == "lm2exp":
            return 2.0 * d["batch"] * d["m"] * d["k"] * d["n"]
        return 2.0 * d["batch"] * d["m"] * d["j"] * d["k"] * d["n"]

    def gbps(self, ms: float) -> float:
        """The reference's metric: input bytes (fp32) over the time."""
        return self.input_elems * 4 * 1e-9 / (ms * 1e-3)

    def make_inputs(self, device, seed: int = 42):
        """`torch.rand` weights and `torch.randn` log-space operands, as the reference's benchmarks draw them."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        d = self.dims
        if self.op == "lm2exp":
            a = torch.rand(d["batch"], d["m"], d["k"], generator=g)
            b = torch.randn(d["batch"], d["k"], d["n"], generator=g)
            return a.to(device), b.to(device)
        w = torch.rand(d["batch"], d["m"], d["j"], d["k"], generator=g)
        a = torch.randn(d["batch"], d["j"], d["n"], generator=g)
        b = torch.randn(d["batch"], d["k"], d["n"], generator=g)
        return w.to(device), a.to(device), b.to(device)


def lm2exp_sweep() -> list[SweepPoint]:
    pts = []
    for x in (128, 192, 256, 384, 512, 768, 1024, 1536, 2048):
        pts.append(SweepPoint("lm2exp", "square, batch=1", dict(batch=1, m=x, k=x, n=x)))
    for batch in (64, 384):
        for x in (64, 96, 128, 192, 256, 384, 512, 768, 1024):
            pts.append(SweepPoint("lm2exp", f"rectangular, n=256 batch={batch}", dict(batch=batch, m=x, k=x, n=256)))
    return pts


def lt2exp_sweep() -> list[SweepPoint]:
    pts = []
    for x in (16, 32, 64, 128, 256, 512):
        pts.append(SweepPoint("lt2exp", "square, batch=1", dict(batch=1, m=x, j=x, k=x, n=x)))
    for batch in (32, 128):
        for x in (16, 32, 64, 128, 256):
            pts.append(SweepPoint("lt2exp", f"rectangular, n=256 batch={batch}", dict(batch=batch, m=x, j=x, k=x, n=256)))
    return pts


SWEEPS = {"lm2exp": lm2exp_sweep, "lt2exp": lt2exp_sweep}

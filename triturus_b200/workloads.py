"""Seeded synthetic inputs for the five benchmark configurations of the lm2exp / lt2exp hot path.

Inputs are generated on the CPU with `torch.Generator().manual_seed(seed)` so that every implementation
under comparison sees identical bits, then moved to the requested device.  The distributions stress the
stabiliser: per-column offsets of up to +-200 and isolated -inf entries.  `scale_r` lets tests run the same
distributions at a smaller batch size.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    op: str          # "lm2exp" or "lt2exp"
    dims: dict       # R, I, J, K (and S for lt2exp)
    description: str

    @property
    def flops(self) -> float:
        d = self.dims
        if self.op == "lm2exp":
            return 2.0 * d["R"] * d["I"] * d["J"] * d["K"]
        return 2.0 * d["R"] * d["S"] * d["I"] * d["J"] * d["K"]

    @property
    def bytes(self) -> float:
        d = self.dims
        if self.op == "lm2exp":
            return 4.0 * d["R"] * (d["I"] * d["J"] + d["J"] * d["K"] + d["I"] * d["K"])
        return 4.0 * d["R"] * (d["S"] * d["I"] * d["J"] + d["I"] * d["K"] + d["J"] * d["K"] + d["S"] * d["K"])

    def with_batch(self, R: int) -> "Workload":
        return Workload(self.name, self.op, {**self.dims, "R": int(R)}, self.description)


WORKLOADS = {
    "cfg1": Workload("cfg1", "lm2exp", dict(R=4, I=256, J=256, K=256),
                     "a ~ U(0,1) normalised over j; b = log_softmax_j(4 N(0,1))"),
    "cfg2": Workload("cfg2", "lm2exp", dict(R=32, I=1024, J=1024, K=1024),
                     "a ~ U(0,1) normalised over j; b ~ N(-20,10) + per-column U(-200,200); 1% -inf"),
    "cfg3": Workload("cfg3", "lm2exp", dict(R=128, I=256, J=256, K=8192),
                     "a = softmax_j N(0,1); b = log_softmax_j(3 N(0,1)) - per-column U(0,50)"),
    "cfg4": Workload("cfg4", "lt2exp", dict(R=16, S=128, I=64, J=64, K=2048),
                     "w ~ U(0,1) normalised over (i,j); a, b = log_softmax(3 N(0,1)) + per-column U(-30,0)"),
    "cfg5": Workload("cfg5", "lt2exp", dict(R=64, S=256, I=128, J=128, K=4096),
                     "w = softmax_(i,j) N(0,1); a, b ~ N(-40,15) with 0.5% -inf"),
}  # fmt: skip


def make_inputs(wl: Workload, seed: int = 0, device: str | torch.device = "cpu") -> tuple[torch.Tensor, ...]:
    """Return (a, b) for lm2exp workloads or (w, a, b) for lt2exp workloads."""
    g = torch.Generator().manual_seed(seed)
    d = wl.dims
    R, I, J, K = d["R"], d["I"], d["J"], d["K"]
    rand = lambda *s: torch.rand(*s, generator=g, dtype=torch.float32)  # noqa: E731
    randn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float32)  # noqa: E731
    ninf = float("-inf")
    if wl.name == "cfg1":
        a = rand(R, I, J)
        a = a / a.sum(-1, keepdim=True)
        b = torch.log_softmax(4.0 * randn(R, J, K), dim=1)
        out = (a, b)
    elif wl.name == "cfg2":
        a = rand(R, I, J)
        a = a / a.sum(-1, keepdim=True)
        b = -20.0 + 10.0 * randn(R, J, K) + (400.0 * rand(R, 1, K) - 200.0)
        b[rand(R, J, K) < 0.01] = ninf
        out = (a, b)
    elif wl.name == "cfg3":
        a = torch.softmax(randn(R, I, J), dim=-1)
        b = torch.log_softmax(3.0 * randn(R, J, K), dim=1) - 50.0 * rand(R, 1, K)
        out = (a, b)
    elif wl.name == "cfg4":
        S = d["S"]
        w = rand(R, S, I, J)
        w = w / w.sum((-2, -1), keepdim=True)
        a = torch.log_softmax(3.0 * randn(R, I, K), dim=1) - 30.0 * rand(R, 1, K)
        b = torch.log_softmax(3.0 * randn(R, J, K), dim=1) - 30.0 * rand(R, 1, K)
        out = (w, a, b)
    elif wl.name == "cfg5":
        S = d["S"]
        w = torch.softmax(randn(R, S, I * J), dim=-1).view(R, S, I, J)
        a = -40.0 + 15.0 * randn(R, I, K)
        a[rand(R, I, K) < 0.005] = ninf
        b = -40.0 + 15.0 * randn(R, J, K)
        b[rand(R, J, K) < 0.005] = ninf
        out = (w, a, b)
    else:
        raise KeyError(wl.name)
    dev = torch.device(device)
    return tuple(t.to(dev) for t in out)

"""lm2exp / lt2exp on HOST tensors: the batch is cut into chunks and the host-to-device copy of chunk c + 1,
the kernels of chunk c and the device-to-host copy of chunk c - 1 run at the same time on three streams.

The reference has no such call (its wrappers take CUDA tensors, triturus/lm2exp.py:167-206,
triturus/lt2exp.py:519-630); a caller that keeps its data in host memory would write
`lm2exp(a.cuda(), b.cuda()).cpu()`, which runs copy-in, kernel and copy-out back to back.  Batch entries are
independent, so the three can overlap: a B200 has separate copy engines for the two directions, and the
kernels are 10-100x shorter than the copies, so a pipelined step costs about the larger of the two copy
times instead of their sum.

Pinned (page-locked) host tensors are needed for the copies to be asynchronous; pageable ones work but
serialise.  The calls return after enqueueing: torch's current stream is made to wait for all three streams,
so `torch.cuda.current_stream().synchronize()` (or any later work on that stream) orders after the result.
"""

from __future__ import annotations

import torch

from .lm2exp import lm2exp
from .lt2exp import lt2exp

# Three private side streams per device: copy in, compute, copy out.
_STREAMS: dict[int, tuple[torch.cuda.Stream, torch.cuda.Stream, torch.cuda.Stream]] = {}

_TARGET_CHUNK_BYTES = 32 << 20  # host-to-device bytes per chunk: long enough to run at full PCIe/C2C rate


def _streams(dev: torch.device):
    st = _STREAMS.get(dev.index)
    if st is None:
        st = tuple(torch.cuda.Stream(device=dev) for _ in range(3))
        _STREAMS[dev.index] = st
    return st


def chunk_bounds(batch: int, bytes_per_entry: int, chunks: int | None = None) -> list[tuple[int, int]]:
    """Cut `batch` entries into contiguous chunks.

    `chunks` given: that many chunks of equal size (at most `batch`).  Otherwise chunks of about 32 MB of input
    with shorter ones at both ends (a quarter, then half of that size): the first copy-in and the last copy-out
    are the only transfers that nothing overlaps, so they are kept short, while the chunks in between are long
    enough to run at the full PCIe / C2C rate."""
    if batch <= 0:
        raise ValueError("empty batch")
    if chunks is not None:
        chunks = max(1, min(int(chunks), batch))
        base, extra = divmod(batch, chunks)
        sizes = [base + (1 if c < extra else 0) for c in range(chunks)]
    else:
        per = max(bytes_per_entry, 1)
        if batch * per < 2 * _TARGET_CHUNK_BYTES:
            sizes = [batch]
        else:
            full = max(1, _TARGET_CHUNK_BYTES // per)
            ramp = [s for s in (max(1, full // 4), max(1, full // 2)) if s < full]
            if 2 * sum(ramp) + full > batch:
                ramp = []
            middle = batch - 2 * sum(ramp)
            n_mid = max(1, min(16, -(-middle // full)))
            base, extra = divmod(middle, n_mid)
            sizes = ramp + [base + (1 if c < extra else 0) for c in range(n_mid)] + ramp[::-1]
    bounds, lo = [], 0
    for size in sizes:
        bounds.append((lo, lo + size))
        lo += size
    return bounds


def _pipelined(op, host_inputs, out_shape, out_host, device, chunks, kwargs):
    for t in host_inputs:
        if t.is_cuda:
            raise ValueError("host entry points take CPU tensors; call lm2exp / lt2exp for CUDA tensors")
        if t.dtype != torch.float32:
            raise AssertionError("operands must be float32")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    if out_host is None:
        out_host = torch.empty(out_shape, dtype=torch.float32, pin_memory=True)
    elif tuple(out_host.shape) != tuple(out_shape) or out_host.dtype != torch.float32 or out_host.is_cuda:
        raise ValueError(f"out must be a float32 CPU tensor of shape {tuple(out_shape)}")
    batch = out_shape[0]
    per_entry = sum(t[0].numel() * 4 for t in host_inputs)
    bounds = chunk_bounds(batch, per_entry, chunks)

    cur = torch.cuda.current_stream(dev)
    if len(bounds) == 1:
        # Nothing to overlap: stay on the current stream and skip the cross-stream events.
        with torch.cuda.stream(cur):
            res = op(*[t.to(dev, non_blocking=True) for t in host_inputs], **kwargs)
            out_host.copy_(res, non_blocking=True)
        return out_host

    s_in, s_run, s_out = _streams(dev)
    start = torch.cuda.Event()
    start.record(cur)
    for s in (s_in, s_run, s_out):
        s.wait_event(start)

    keep = []  # device tensors stay referenced until every stream has been joined
    for lo, hi in bounds:
        with torch.cuda.stream(s_in):
            dev_in = [t[lo:hi].to(dev, non_blocking=True) for t in host_inputs]
            copied = torch.cuda.Event()
            copied.record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(copied)
            res = op(*dev_in, **kwargs)
            done = torch.cuda.Event()
            done.record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            out_host[lo:hi].copy_(res, non_blocking=True)
        keep.append((dev_in, res))
    for s in (s_in, s_run, s_out):
        ev = torch.cuda.Event()
        ev.record(s)
        cur.wait_event(ev)
    for dev_in, res in keep:
        for t in (*dev_in, res):
            t.record_stream(cur)
    return out_host


def lm2exp_host(a: torch.Tensor, b: torch.Tensor, *, out: torch.Tensor | None = None, device=None,
                chunks: int | None = None, precision: str | None = None, variant: int = 0) -> torch.Tensor:
    """lm2exp for host tensors a [R,I,J], b [R,J,K]; returns (or fills) a pinned host tensor [R,I,K].
    Same checks and results as `lm2exp`; every chunk of the batch runs the same kernels."""
    assert len(a.shape) == len(b.shape) == 3
    assert a.shape[0] == b.shape[0]
    assert a.shape[2] == b.shape[1]
    kwargs = {"precision": precision, "variant": variant}
    return _pipelined(lm2exp, (a, b), (a.shape[0], a.shape[1], b.shape[2]), out, device, chunks, kwargs)


def lt2exp_host(w: torch.Tensor, a: torch.Tensor, b: torch.Tensor, *, out: torch.Tensor | None = None, device=None,
                chunks: int | None = None, mode: str = "auto", precision: str | None = None,
                variant: int = 0) -> torch.Tensor:
    """lt2exp for host tensors w [R,S,I,J], a [R,I,K], b [R,J,K]; returns (or fills) a pinned host tensor
    [R,S,K]."""
    assert len(w.shape) == 4
    assert len(a.shape) == len(b.shape) == 3
    assert w.shape[0] == a.shape[0] == b.shape[0]
    assert w.shape[2] == a.shape[1]
    assert w.shape[3] == b.shape[1]
    assert a.shape[2] == b.shape[2]
    kwargs = {"mode": mode, "precision": precision, "variant": variant}
    return _pipelined(lt2exp, (w, a, b), (w.shape[0], w.shape[1], a.shape[2]), out, device, chunks, kwargs)

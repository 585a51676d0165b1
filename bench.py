#!/usr/bin/env python
"""Benchmark of the lm2exp / lt2exp hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--precision tf32] [--impl ours]

A "step" is one pass of the op over one batch of synthetic input.  At N = 1 the workload is cfg2
(lm2exp fp32, R=32, I=J=K=1024, the configuration the headline metric is quoted on).  For N > 1 the script
is launched once per GPU by torch.distributed.run; the batch dimension is the sharded unit and every rank
holds one full copy of the workload's batch (weak scaling, no collective on the data path).  Rank 0 prints
one JSON line.

`value` is device-timed (CUDA events, max over ranks) with inputs resident in HBM.  `e2e` is the same
metric through the public Python entry point starting from pinned host tensors, with the host-to-device
copy of the operands and the device-to-host copy of the result inside the timed region.
`--impl reference` times the reference's CPU path (its torch baseline, restated in oracle/) on the host
cores instead.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from triturus_b200.workloads import WORKLOADS, make_inputs  # noqa: E402

METRIC = "lm2exp/lt2exp effective TFLOP/s"


def launches_per_step(wl, precision: str, variant: int, chain: bool = False) -> int:
    """Kernels of this library launched per step, asked from the library: lm2exp is the contraction kernel
    plus, unless the max pass is fused into it, the stabiliser pre-pass; lt2exp is one kernel, or three
    (zero-fill, contraction slices, log pass) when the contraction is split over the SMs."""
    from triturus_b200 import _native

    d = wl.dims
    prec = 0 if precision == "tf32" else 1
    if wl.op == "lt2exp":
        n = _native.LIB.triturus_b200_lt2exp_launches(d["R"], d["S"], d["I"], d["J"], d["K"], prec, variant)
    elif chain:
        n = _native.LIB.triturus_b200_lm2exp_chain_launches(d["R"], d["I"], d["J"], d["K"], prec, variant, 1, 1)
    else:
        n = _native.LIB.triturus_b200_lm2exp_launches(d["R"], d["I"], d["J"], d["K"], prec, variant)
    if n <= 0:
        raise RuntimeError(f"launch-count query returned {n}")
    return int(n)

# DRAM traffic per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum) taken from
# the committed ncu summaries under profiles/; None where no capture exists yet.
NCU_TRAFFIC_BYTES = {
    ("cfg2", "tf32"): 271.47e6 + 102.55e6,   # profiles/lm2exp_pair_kernel_cfg2.md
    ("cfg3", "tf32"): 1107.47e6 + 1024.21e6,  # profiles/lm2exp_kernel_cfg3.md
    ("cfg5", "tf32"): 1999.31e6 + 237.76e6,   # profiles/lt2exp_kernel_cfg5.md
}


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {
            "hbm_gbs": float(d["hbm_gbs"]),
            "bf16_tflops": float(d["bf16_tflops"]),
            "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
            "source": "measured",
        }
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""

    FIELDS = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )  # fmt: skip
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = sorted(sm)[len(sm) // 2 :]  # upper half: samples taken under load
        return {
            "sm_mhz": statistics.median(busy),
            "sm_max_mhz": max(sm_max),
            "reasons": sorted(reasons),
            "samples": len(sm),
        }


def dist_env() -> tuple[int, int, int]:
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def make_step(op_name: str, precision: str, variant: int):
    import triturus_b200 as tb

    op = tb.lm2exp if op_name == "lm2exp" else tb.lt2exp
    return lambda *xs: op(*xs, precision=precision, variant=variant)


def cpu_reference_time(wl, reps: int, warmup: int = 1) -> tuple[float, int, str]:
    """Median seconds per full pass of the reference's CPU path (oracle restatement of
    baselines/lm2exp.py / baselines/lt2exp.py) on a bounded sample of the workload."""
    from oracle import logspace_oracle as orc

    sample = wl
    note = "full workload"
    # One batch entry of cfg5 needs a 1 GiB Khatri-Rao intermediate on the CPU; bound the sample.
    if wl.op == "lt2exp" and wl.dims["I"] * wl.dims["J"] * wl.dims["K"] * wl.dims["R"] > (1 << 31):
        sample = wl.with_batch(2)
        note = f"R=2 of {wl.dims['R']} batch entries, time scaled by {wl.dims['R'] / 2:g}"
    # torchrun exports OMP_NUM_THREADS=1; the CPU baseline uses every core this process may run on.
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    xs = make_inputs(sample, seed=0)
    fn = orc.lm2exp_fp32 if wl.op == "lm2exp" else orc.lt2exp_fp32
    for _ in range(warmup):
        fn(*xs)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn(*xs)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times) * (wl.dims["R"] / sample.dims["R"])
    return sec, torch.get_num_threads(), f"{note}; median of {reps} runs after {warmup} warm-up"


def run_reference_arm(args, wl) -> None:
    rank, _, world = dist_env()
    if rank != 0:
        return
    steps = max(1, args.steps)
    sec, cores, sample = cpu_reference_time(wl, reps=min(steps, 5), warmup=min(max(args.warmup, 1), 2))
    tflops = wl.flops / sec / 1e12
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": tflops,
        "unit": "TFLOP/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": sec * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"{wl.name}: {wl.op} fp32 {wl.dims}", "where": "host CPU, torch (MKL) baseline"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_sweep(args) -> None:
    """The reference's benchmark sweeps (benchmarks/lm2exp.py, benchmarks/lt2exp.py) on one GPU: one JSON line
    per shape and TF32 setting with the reference's GB/s (input bytes only) beside TFLOP/s, for this library
    and for the same formula written with torch ops on the GPU (cuBLAS bmm), the reference's "torch" provider."""
    import triturus_b200 as tb
    from triturus_b200.sweeps import SWEEPS
    from triturus_b200.utils import set_tf32_enabled

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)

    def torch_provider(op):
        def lm(a, b):
            m = b.amax(dim=1, keepdim=True).clamp(-1e38, 1e38)
            return m + torch.bmm(a, (b - m).exp()).log()

        def lt(w, a, b):
            ma = a.amax(dim=1, keepdim=True).clamp(-1e38, 1e38)
            mb = b.amax(dim=1, keepdim=True).clamp(-1e38, 1e38)
            kr = ((a - ma).exp()[:, :, None, :] * (b - mb).exp()[:, None, :, :]).flatten(1, 2)
            return ma + mb + torch.bmm(w.flatten(2, 3), kr).log()

        return lm if op == "lm2exp" else lt

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # written between timed calls: cold L2

    def median_ms(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        for e0, e1 in evs:
            flush.zero_()
            e0.record()
            fn()
            e1.record()
        torch.cuda.synchronize()
        return statistics.median(e0.elapsed_time(e1) for e0, e1 in evs)

    ours = tb.lm2exp if args.sweep == "lm2exp" else tb.lt2exp
    ref = torch_provider(args.sweep)
    for allow_tf32 in (False, True):
        set_tf32_enabled(allow_tf32)
        for pt in SWEEPS[args.sweep]():
            xs = pt.make_inputs(dev)
            ms = median_ms(lambda: ours(*xs), args.steps)
            ms_t = median_ms(lambda: ref(*xs), max(3, args.steps // 4))
            print(json.dumps({
                "sweep": f"{pt.op} ({pt.family}, allow_tf32={allow_tf32})", "dims": pt.dims,
                "triturus_b200": {"ms": ms, "GB/s": pt.gbps(ms), "TFLOP/s": pt.flops / ms / 1e9},
                "torch": {"ms": ms_t, "GB/s": pt.gbps(ms_t), "TFLOP/s": pt.flops / ms_t / 1e9},
            }), flush=True)  # fmt: skip
    set_tf32_enabled(False)
    tb.check_status()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="cfg2")
    ap.add_argument("--precision", choices=["tf32", "3xtf32"], default="tf32")
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-mode", action="store_true",
                    help="only W warm-up and K timed steps: no clock sampling, end-to-end leg or CPU baseline "
                         "(for runs under a profiler, whose printed numbers are never bench values)")
    ap.add_argument("--chain", action="store_true",
                    help="lm2exp workloads: time one inner link of a chain of layers (the stabiliser of b is "
                         "supplied, the column maxima of the result are returned); not the headline configuration")
    ap.add_argument("--gather", action="store_true", help="also time an all-gather of the output shards (reported separately)")
    ap.add_argument("--sweep", choices=["lm2exp", "lt2exp"], default=None,
                    help="walk the reference's benchmark sweep for one op instead of the headline workload")
    ap.add_argument("--dims", default=None,
                    help="override dimensions of the chosen workload, e.g. R=1,S=512,I=512,J=512,K=512 "
                         "(same input distribution; for profiling other shapes, not a headline number)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    custom_dims = False
    if args.dims:
        over = {k.strip(): int(v) for k, v in (kv.split("=") for kv in args.dims.split(","))}
        unknown = set(over) - set(wl.dims)
        if unknown:
            raise SystemExit(f"--dims: {sorted(unknown)} are not dimensions of {wl.name} ({sorted(wl.dims)})")
        wl = type(wl)(wl.name, wl.op, {**wl.dims, **over}, wl.description)
        custom_dims = True

    if args.sweep is not None:
        run_sweep(args)
        return

    if args.impl == "reference":
        run_reference_arm(args, wl)
        return

    rank, local_rank, world = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    import triturus_b200 as tb

    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    step = make_step(wl.op, args.precision, args.variant)
    if args.chain and wl.op != "lm2exp":
        raise SystemExit("--chain applies to the lm2exp workloads")

    # Weak scaling: every rank owns one full batch of the workload (seeded per rank).
    host_inputs = [t.pin_memory() for t in make_inputs(wl, seed=rank)]
    inputs = [t.to(dev, non_blocking=True) for t in host_inputs]
    torch.cuda.synchronize()
    if args.chain:
        # Steady state of a chain: the previous layer's epilogue delivered the column maxima of b.
        b_colmax = tb.colmax(inputs[1])
        step = lambda a, b: tb.lm2exp(a, b, precision=args.precision, variant=args.variant,  # noqa: E731
                                      b_colmax=b_colmax, return_colmax=True)[0]

    def barrier() -> None:
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- device-resident timing
    for _ in range(warmup):
        out = step(*inputs)
    tb.check_status()
    # The timed region can be a few milliseconds, shorter than one nvidia-smi sampling period, so the same
    # step keeps the GPU loaded (untimed) until the sampler has delivered samples before the timed region
    # and for a short while after it; the reported clock is the median of the samples under that load.
    sampler = ClockSampler(local_rank)
    if not args.profile_mode:
        sampler.start()
    lead_in_deadline = time.perf_counter() + (0.0 if args.profile_mode else 4.0)
    while len(sampler.lines) < 3 and time.perf_counter() < lead_in_deadline:
        for _ in range(8):
            out = step(*inputs)
        torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    # Workloads whose operands and result fit in the 126 MB L2 (cfg1, cfg4) get the L2 flushed between timed
    # steps by writing a 256 MB buffer; the others evict themselves.
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if wl.bytes < 2 * 126e6 else None
    barrier()
    t_wall0 = time.perf_counter()
    for e0, e1 in evs:
        if flush is not None:
            flush.zero_()
        e0.record()
        out = step(*inputs)
        e1.record()
    barrier()
    t_wall = time.perf_counter() - t_wall0
    n_before = len(sampler.lines)
    lead_out_deadline = time.perf_counter() + (0.0 if args.profile_mode else 1.5)
    while len(sampler.lines) < n_before + 3 and time.perf_counter() < lead_out_deadline:
        for _ in range(8):
            out = step(*inputs)
        torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["note"] = "sampled every 200 ms while the timed step ran back to back before, during and after the timed region"
    tb.check_status()
    per_step_ms = [e0.elapsed_time(e1) for e0, e1 in evs]
    # With a flush between steps only the bracketed step times count; otherwise first start to last end.
    total_ms = sum(per_step_ms) if flush is not None else evs[0][0].elapsed_time(evs[-1][1])
    t = torch.tensor([total_ms, sum(per_step_ms) / steps], device=dev, dtype=torch.float64)
    if distributed:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, launch_ms = float(t[0]), float(t[1])
    ms_per_step = total_ms / steps
    value = world * wl.flops / (ms_per_step * 1e-3) / 1e12

    if args.profile_mode:
        if rank == 0:
            print(json.dumps({"profile_mode": True, "workload": wl.name, "ms_per_step": ms_per_step,
                              "note": "not a bench value"}), flush=True)  # fmt: skip
        if distributed:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---------------------------------------------------------------- end to end from pinned host memory
    # The call a user with host-resident data makes: the pipelined host entry point (copy-in, kernels and
    # copy-out of successive batch chunks overlap on three streams); every byte still crosses the bus inside
    # the timed region.
    host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    e2e_steps = max(3, min(steps, 10))
    host_fn = tb.lm2exp_host if wl.op == "lm2exp" else tb.lt2exp_host

    def e2e_step() -> None:
        host_fn(*host_inputs, out=host_out, precision=args.precision, variant=args.variant)

    for _ in range(2):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if distributed:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t[0]) / e2e_steps
    e2e_value = world * wl.flops / (e2e_ms * 1e-3) / 1e12
    h2d = sum(t.numel() * t.element_size() for t in host_inputs)
    d2h = host_out.numel() * host_out.element_size()

    # ---------------------------------------------------------------- optional all-gather, reported apart
    gather_ms = None
    if args.gather and distributed:
        full = torch.empty((world * out.shape[0], *out.shape[1:]), dtype=out.dtype, device=dev)
        for _ in range(2):
            dist.all_gather_into_tensor(full, out)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(5):
            dist.all_gather_into_tensor(full, out)
        g1.record()
        barrier()
        t = torch.tensor([g0.elapsed_time(g1) / 5], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gather_ms = float(t[0])

    # lm2exp with a pre-pass launches two kernels per step; the roofline is that of the dominant one (the
    # contraction kernel), so the stabiliser pre-pass is timed on its own and taken off the step time.
    n_launch = launches_per_step(wl, args.precision, args.variant, args.chain)
    prepass_ms = 0.0
    if wl.op == "lm2exp" and n_launch == 2 and not args.chain:
        for _ in range(3):
            tb.colmax(inputs[1])
        pe = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        torch.cuda.synchronize()
        for e0, e1 in pe:
            if flush is not None:
                flush.zero_()  # same cold L2 as the timed steps; the fill also hides the host side of the call
            e0.record()
            tb.colmax(inputs[1])
            e1.record()
        torch.cuda.synchronize()
        prepass_ms = statistics.median(e0.elapsed_time(e1) for e0, e1 in pe)
        if prepass_ms >= 0.9 * launch_ms:
            # A step this short is launch latency, not kernel time: leave the step time undivided.
            prepass_ms = 0.0
    launch_ms = max(launch_ms - prepass_ms, 1e-6)

    if rank == 0:
        peaks = load_peaks()
        tensor_bound = wl.name in ("cfg2", "cfg4", "cfg5")
        if tensor_bound:
            # Dense TF32 runs at half the bf16 rate; the bf16 figure is the measured cuBLAS burst number.
            peak = peaks["bf16_tflops"] / 2.0
            achieved = wl.flops / (launch_ms * 1e-3) / 1e12
            # Two measured cuBLAS figures exist: a burst (best of ten isolated GEMMs) and a sustained one (GEMMs
            # back to back for seconds, SM clock pulled down by the 1 kW power cap).  The timed region here is
            # a loop of steps preceded by seconds of the same load, so when the clock samples taken during it
            # report sw_power_cap the kernel ran in the sustained regime and that figure is the denominator;
            # otherwise the burst figure is.  Both fractions are reported.
            burst = peaks["bf16_tflops"] / 2.0
            sustained = peaks["bf16_tflops_sustained"] / 2.0
            capped = "sw_power_cap" in clocks.get("reasons", [])
            peak = sustained if capped else burst
            achieved = wl.flops / (launch_ms * 1e-3) / 1e12
            roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak,
                    "peak_source": (f"0.5 x bf16 cuBLAS {'sustained (timed under sw_power_cap)' if capped else 'burst'}, "
                                    f"{peaks['source']}"),
                    "frac_of_burst": achieved / burst, "frac_of_sustained": achieved / sustained}  # fmt: skip
        else:
            peak = peaks["hbm_gbs"]
            achieved = wl.bytes / (launch_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "peak_source": f"stream copy, {peaks['source']}"}  # fmt: skip
        roof["traffic"] = None if custom_dims else NCU_TRAFFIC_BYTES.get((wl.name, args.precision))
        roof["launch_ms"] = launch_ms
        roof["prepass_ms"] = prepass_ms
        roof["kernel"] = ("lt2exp_kernel" if wl.op == "lt2exp" else
                          "lm2exp chain link (stabiliser supplied, column maxima returned)" if args.chain else
                          ("lm2exp_pair_kernel / lm2exp_kernel (step time minus the stabiliser pre-pass)" if n_launch == 2
                           else "lm2exp_kernel (fused max pass)"))

        line = {
            "metric": METRIC,
            "value": value,
            "unit": "TFLOP/s",
            "n_gpus": world,
            "steps": steps,
            "warmup": warmup,
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "tf32" if args.precision == "tf32" else "3xtf32",
            "data": "synthetic",
            "config": {
                "workload": f"{wl.name}{' (custom dims)' if custom_dims else ''}: {wl.op} fp32 {wl.dims} per GPU",
                "precision": args.precision,
                "variant": args.variant,
                **({"chain": "inner link: b_colmax supplied, out_colmax returned"} if args.chain else {}),
                "sharding": f"batch r, one full batch per GPU x {world}",
                "l2": (f"operands + result = {wl.bytes / 1e6:.0f} MB per step, larger than the 126 MB L2"
                       if flush is None else
                       f"operands + result = {wl.bytes / 1e6:.0f} MB per step fit in the 126 MB L2: "
                       "a 256 MB buffer is written between timed steps"),
            },
            "roofline": roof,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "steps": e2e_steps},  # fmt: skip
            "gpu_launches": n_launch * steps,
            "clocks": clocks,
            "wall_s": t_wall,
        }
        if gather_ms is not None:
            line["all_gather_ms"] = gather_ms
        if world == 1 and not args.no_cpu_baseline:
            sec, cores, sample = cpu_reference_time(wl, reps=5 if wl.name != "cfg5" else 1)
            line["cpu_baseline"] = {"value": wl.flops / sec / 1e12, "unit": "TFLOP/s", "cores": cores,
                                    "kind": "port", "sample": sample}  # fmt: skip
        print(json.dumps(line), flush=True)

    if distributed:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

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

`roofline.frac` is the whole step (every kernel a call launches) over the measured peak; the contraction
kernel alone, timed directly with its stabiliser supplied, is `roofline.frac_dominant_kernel`.  Every line
also carries `strong_cfg5`: lt2exp cfg5 (R = 64) cut into R / N batch entries per rank, the strong-scaling
figure of the largest configuration.  At N = 1 the line adds `configs` (the other four configurations), a
cuBLAS TF32 figure measured in the same run, the reference's Triton kernel on the same inputs (when
baseline/_ref holds the reference) and the CPU baselines.

`--impl reference` times the reference's CPU path (its torch baselines from baseline/_ref when present, else
their restatement in oracle/) on the host cores instead; it imports nothing of this library.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

# torch.compile's CPU code (the reference's jit baselines) is built with $CXX, read when torch's inductor
# configuration is first imported; it needs a g++ that finds its OpenMP runtime, which the system one does.
if os.path.exists("/usr/bin/g++"):
    os.environ["CXX"] = "/usr/bin/g++"

import torch  # noqa: E402

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _load_workloads():
    """The workload definitions, loaded from their file so that the reference arm does not import the
    package (whose __init__ maps the CUDA library into the process)."""
    name = "_tb200_workloads"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, ROOT / "triturus_b200" / "workloads.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


_wl = _load_workloads()
WORKLOADS, make_inputs = _wl.WORKLOADS, _wl.make_inputs

METRIC = "lm2exp/lt2exp effective TFLOP/s"
TENSOR_BOUND = ("cfg2", "cfg4", "cfg5")
SM_COUNT, TF32_MAC_PER_CLK_SM = 148, 2048  # dense tf32 tcgen05 rate per SM and clock


def workload_string(wl, custom: bool = False) -> str:
    return f"{wl.name}{' (custom dims)' if custom else ''}: {wl.op} fp32 {wl.dims}"


def launches_per_step(wl, precision: str, variant: int, chain: bool = False) -> int:
    """Kernels of this library launched per step, asked from the library: lm2exp is the contraction kernel
    plus, unless the max pass is fused into it, the stabiliser pre-pass; lt2exp is one kernel, or three
    (zero-fill, contraction, log pass) when the contraction is split over the SMs."""
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


def plan_code(wl, precision: str, variant: int) -> int:
    """The explicit variant code of what the library runs for this workload (tile shape, stabiliser / split form)."""
    from triturus_b200 import _native

    d = wl.dims
    prec = 0 if precision == "tf32" else 1
    if wl.op == "lt2exp":
        return int(_native.LIB.triturus_b200_lt2exp_plan(d["R"], d["S"], d["I"], d["J"], d["K"], prec, variant))
    return int(_native.LIB.triturus_b200_lm2exp_plan(d["R"], d["I"], d["J"], d["K"], prec, variant))


# DRAM traffic per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum) taken from
# the committed ncu summaries under profiles/; None where no capture exists.
NCU_TRAFFIC_BYTES = {
    ("cfg2", "tf32"): 272.34e6 + 100.83e6,   # profiles/lm2exp_tspair_kernel_cfg2.md
    ("cfg3", "tf32"): 1107.41e6 + 1016.16e6,  # profiles/lm2exp_tspair_kernel_cfg3.md
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
        sm, sm_max, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # Every sample is taken while the timed step runs back to back (lead-in, timed region, lead-out), so
        # the plain median over all of them is the clock under load.
        return {
            "sm_mhz": statistics.median(sm),
            "sm_mhz_min": min(sm),
            "sm_mhz_max": max(sm),
            "sm_max_mhz": max(sm_max),
            "power_w_median": statistics.median(power) if power else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }


def dist_env() -> tuple[int, int, int]:
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def bind_to_gpu_numa_node(local_rank: int) -> dict:
    """Restrict this process to the cores of the NUMA node its GPU hangs off, before any pinned host buffer is
    allocated (page-locked memory is placed on the node of the allocating thread).  Launchers such as
    torch.distributed.run do not bind ranks, so without this the pinned buffers of half the ranks can sit on
    the far socket and every host copy crosses the socket interconnect."""
    info: dict = {"numa_node": None}
    try:
        props = torch.cuda.get_device_properties(local_rank)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        node = int(Path(f"/sys/bus/pci/devices/{bdf}/numa_node").read_text().strip())
        info["pci"] = bdf
        if node < 0:
            info["why"] = "the platform reports no NUMA node for this device"
            return info
        cpus: set[int] = set()
        for part in Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            info["why"] = "none of the node's cores is in this process's affinity mask"
            return info
        os.sched_setaffinity(0, allowed)
        info.update(numa_node=node, cores=len(allowed))
    except Exception as exc:  # noqa: BLE001  (no sysfs, no such attribute: run unbound)
        info["why"] = f"{type(exc).__name__}: {exc}"
    return info


def make_step(op_name: str, precision: str, variant: int):
    import triturus_b200 as tb

    op = tb.lm2exp if op_name == "lm2exp" else tb.lt2exp
    return lambda *xs: op(*xs, precision=precision, variant=variant)


# ------------------------------------------------------------------------------------------ CPU baselines


def _reference_baselines():
    """The reference's own torch baselines (eager and torch.compile forms) when baseline/_ref holds them."""
    suite = ROOT / "baseline" / "_ref" / "suite"
    if not (suite / "baselines" / "lm2exp.py").exists():
        return None
    sys.path.insert(0, str(suite))
    try:
        from baselines import lm2exp as bl_lm  # noqa: PLC0415
        from baselines import lt2exp as bl_lt  # noqa: PLC0415
    finally:
        sys.path.remove(str(suite))
    return {"lm2exp": (bl_lm.lm2exp, bl_lm.lm2exp_jit), "lt2exp": (bl_lt.lt2exp, bl_lt.lt2exp_jit)}


def cpu_reference_time(wl, reps: int, warmup: int = 1, jit: bool = False) -> dict:
    """Median seconds per full pass of the reference's CPU path on a bounded sample of the workload: the
    reference's baselines/lm2exp.py / baselines/lt2exp.py when baseline/_ref holds them ("reference"), else
    their restatement in oracle/ ("port")."""
    ref = _reference_baselines()
    if ref is not None:
        fn = ref[wl.op][1 if jit else 0]
        kind = "reference"
    else:
        from oracle import logspace_oracle as orc

        fn = orc.lm2exp_fp32 if wl.op == "lm2exp" else orc.lt2exp_fp32
        if jit:
            fn = torch.compile(fn)
        kind = "port"
    sample = wl
    note = "full workload"
    # One batch entry of cfg5 needs a 1 GiB Khatri-Rao intermediate on the CPU; bound the sample.
    if wl.op == "lt2exp" and wl.dims["I"] * wl.dims["J"] * wl.dims["K"] * wl.dims["R"] > (1 << 31):
        sample = wl.with_batch(2)
        note = f"R=2 of {wl.dims['R']} batch entries, time scaled by {wl.dims['R'] / 2:g}"
    # torchrun exports OMP_NUM_THREADS=1; the CPU baseline uses every core this process may run on.
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    xs = make_inputs(sample, seed=0)
    for _ in range(warmup):
        fn(*xs)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn(*xs)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times) * (wl.dims["R"] / sample.dims["R"])
    return {"value": wl.flops / sec / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"{note}; median of {reps} runs after {warmup} warm-up; torch {'compile' if jit else 'eager'} (MKL)",
            "ms": sec * 1e3}  # fmt: skip


def run_reference_arm(args, wl) -> None:
    rank, _, world = dist_env()
    if rank != 0:
        return
    steps = max(1, args.steps)
    base = cpu_reference_time(wl, reps=min(steps, 5), warmup=min(max(args.warmup, 1), 2))
    tflops, ms = base["value"], base.pop("ms")
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": tflops,
        "unit": "TFLOP/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_string(wl), "where": "host CPU, the reference's torch baseline"},
        "cpu_baseline": base,
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    try:
        jit = cpu_reference_time(wl, reps=min(steps, 3), warmup=1, jit=True)
        jit.pop("ms")
        line["cpu_baseline_jit"] = jit
    except Exception as exc:  # noqa: BLE001
        line["cpu_baseline_jit"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ sweeps


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


# ------------------------------------------------------------------------------------------ timing helpers


def quantiles(xs: list[float]) -> dict:
    s = sorted(xs)
    pick = lambda q: s[min(len(s) - 1, max(0, int(round(q * (len(s) - 1)))))]  # noqa: E731
    return {"n": len(s), "p10": pick(0.1), "p50": pick(0.5), "p90": pick(0.9), "min": s[0], "max": s[-1]}


def time_steps(fn, steps: int, flush) -> list[float]:
    """CUDA-event time of each of `steps` calls of fn on the current stream (ms); a 256 MB buffer is written
    before every call when `flush` is given."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for e0, e1 in evs:
        if flush is not None:
            flush.zero_()
        e0.record()
        fn()
        e1.record()
    torch.cuda.synchronize()
    return [e0.elapsed_time(e1) for e0, e1 in evs]


def roofline_of(wl, ms: float, peaks: dict, clocks: dict | None) -> dict:
    """Roofline fractions of one step of `wl` that took `ms`, every kernel of the step included."""
    if wl.name in TENSOR_BOUND:
        achieved = wl.flops / (ms * 1e-3) / 1e12
        burst, sustained = peaks["bf16_tflops"] / 2.0, peaks["bf16_tflops_sustained"] / 2.0
        sm_mhz = (clocks or {}).get("sm_mhz")
        sm_max = (clocks or {}).get("sm_max_mhz")
        # Which measured cuBLAS figure applies follows from the clock the step ran at, not from a flag: the
        # burst figure was taken at (nearly) the full clock, the sustained one under the power cap.
        capped = bool(sm_mhz and sm_max and sm_mhz < 0.9 * sm_max)
        peak = sustained if capped else burst
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": (f"0.5 x bf16 cuBLAS {'sustained' if capped else 'burst'} ({peaks['source']}); "
                                f"chosen by the median sampled SM clock {sm_mhz} of {sm_max} MHz"),
                "frac_of_burst": achieved / burst, "frac_of_sustained": achieved / sustained}  # fmt: skip
        if sm_mhz:
            clock_peak = SM_COUNT * TF32_MAC_PER_CLK_SM * 2 * sm_mhz * 1e6 / 1e12
            roof["clock_peak"] = clock_peak  # 148 SMs x 2048 tf32 MAC per clock x 2 at the sampled clock
            roof["frac_of_clock_peak"] = achieved / clock_peak
        return roof
    achieved = wl.bytes / (ms * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"], "peak_source": f"stream copy ({peaks['source']})"}  # fmt: skip


def cublas_tf32_tflops(dev) -> dict:
    """cuBLAS TF32 on this device, in this run: torch.bmm on the cfg2 shape and a square 8192 GEMM."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    out = {}
    try:
        for name, shape_a, shape_b, flops in (
            ("bmm_32x1024x1024x1024", (32, 1024, 1024), (32, 1024, 1024), 2.0 * 32 * 1024**3),
            ("mm_8192", (8192, 8192), (8192, 8192), 2.0 * 8192**3),
        ):
            a = torch.randn(*shape_a, device=dev)
            b = torch.randn(*shape_b, device=dev)
            fn = (lambda: torch.bmm(a, b)) if len(shape_a) == 3 else (lambda: torch.mm(a, b))
            for _ in range(5):
                fn()
            torch.cuda.synchronize()
            ms = statistics.median(time_steps(fn, 30, None))
            out[name] = flops / (ms * 1e-3) / 1e12
            del a, b
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    return out


def triton_reference_times(wl, inputs, steps: int, flush) -> dict:
    """The reference's own Triton kernel (baseline/_ref) on the same device tensors, after its autotuner has
    settled: median ms with its TF32 flag on and off.  lt2exp runs mode="unsplit" (the split kernel's merge is
    a spin lock without a bound and is never launched here)."""
    from baseline import reference_loader as rl

    why = rl.available()
    if why is not None:
        return {"unavailable": why}
    out: dict = {}
    try:
        ref = rl.load()
        fn = (lambda: ref.lm2exp(*inputs)) if wl.op == "lm2exp" else (lambda: ref.lt2exp(*inputs, mode="unsplit"))
        for allow in (True, False):
            ref.set_tf32_enabled(allow)
            try:
                for _ in range(3):  # the first call autotunes
                    fn()
                torch.cuda.synchronize()
                ms = statistics.median(time_steps(fn, steps, flush))
            finally:
                ref.set_tf32_enabled(False)
            out["tf32" if allow else "ieee"] = {"ms": ms, "TFLOP/s": wl.flops / (ms * 1e-3) / 1e12}
    except Exception as exc:  # noqa: BLE001
        out["unavailable"] = f"{type(exc).__name__}: {str(exc)[:300]}"
    return out


def strong_cfg5_inputs(lo: int, hi: int, dev):
    """Batch entries [lo, hi) of cfg5, each generated from its own seed so that the full batch is the same
    whatever the number of ranks."""
    one = WORKLOADS["cfg5"].with_batch(1)
    parts = [make_inputs(one, seed=5000 + r) for r in range(lo, hi)]
    return [torch.cat([p[i] for p in parts], dim=0).to(dev) for i in range(3)]


# ------------------------------------------------------------------------------------------ main


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
    ap.add_argument("--no-extras", action="store_true",
                    help="only the contract's keys: no strong_cfg5 / configs / cuBLAS / Triton / 3xTF32 legs")
    ap.add_argument("--triton-ref", choices=["none", "workload", "all"], default="workload",
                    help="time the reference's Triton kernel (baseline/_ref) on the workload; 'all' adds a cfg5 sample")
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
    all_cores = os.sched_getaffinity(0)
    numa = bind_to_gpu_numa_node(local_rank)
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    import triturus_b200 as tb
    from triturus_b200.sharding import shard_bounds

    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    step = make_step(wl.op, args.precision, args.variant)
    if args.chain and wl.op != "lm2exp":
        raise SystemExit("--chain applies to the lm2exp workloads")
    extras = not (args.no_extras or args.profile_mode or custom_dims or args.chain)

    def rank_max(*vals: float) -> list[float]:
        t = torch.tensor(vals, device=dev, dtype=torch.float64)
        if distributed:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

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
    per_step_ms = [e0.elapsed_time(e1) for e0, e1 in evs]
    # With a flush between steps only the bracketed step times count; otherwise first start to last end.
    total_ms = sum(per_step_ms) if flush is not None else evs[0][0].elapsed_time(evs[-1][1])
    # Quantiles over at least 100 launches: the timed steps plus as many more of the same, still under load.
    more = [] if args.profile_mode else time_steps(lambda: step(*inputs), max(0, 100 - steps), flush)
    # The dominant kernel alone, timed directly: for lm2exp with a stabiliser pre-pass, the contraction kernel
    # with the column maxima supplied (it is then the only launch of the call) and the pre-pass by itself.
    n_launch = launches_per_step(wl, args.precision, args.variant, args.chain)
    kernel_ms = prepass_ms = None
    pcode = plan_code(wl, args.precision, args.variant)
    # 0 optimistic TMEM-operand pair kernel, 1 pre-pass, 2 / 3 fused max pass, 4 optimistic 32-row pre-pass
    stab = pcode // 100000 if wl.op == "lm2exp" else -1
    if stab in (0, 1, 4) and not args.chain and not args.profile_mode:
        m_pre = tb.colmax(inputs[1])
        kern = lambda: tb.lm2exp(*inputs, precision=args.precision, variant=args.variant, b_colmax=m_pre)  # noqa: E731
        for _ in range(3):
            kern()
        kernel_ms = statistics.median(time_steps(kern, max(20, min(steps, 100)), flush))
        if stab == 1:  # (the optimistic forms have no full pre-pass in the step)
            prepass_ms = statistics.median(time_steps(lambda: tb.colmax(inputs[1]), max(20, min(steps, 100)), flush))
    n_before = len(sampler.lines)
    lead_out_deadline = time.perf_counter() + (0.0 if args.profile_mode else 1.5)
    while len(sampler.lines) < n_before + 3 and time.perf_counter() < lead_out_deadline:
        for _ in range(8):
            out = step(*inputs)
        torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["note"] = "sampled every 200 ms while the timed step ran back to back before, during and after the timed region"
    tb.check_status()
    total_ms, launch_ms = rank_max(total_ms, sum(per_step_ms) / steps)
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
    my_e2e_ms = e0.elapsed_time(e1) / e2e_steps
    (e2e_ms,) = rank_max(my_e2e_ms)
    e2e_value = world * wl.flops / (e2e_ms * 1e-3) / 1e12
    h2d = sum(t.numel() * t.element_size() for t in host_inputs)
    d2h = host_out.numel() * host_out.element_size()
    # Host copies alone, per rank, all ranks at once: what the host side of the box delivers.
    h2d_copy = lambda: [d.copy_(h, non_blocking=True) for d, h in zip(inputs, host_inputs)]  # noqa: E731
    h2d_copy()
    barrier()
    my_h2d_gbs = h2d / (statistics.median(time_steps(h2d_copy, 5, None)) * 1e-3) / 1e9
    copy_rates = torch.tensor([my_h2d_gbs, my_e2e_ms], device=dev, dtype=torch.float64)
    if distributed:
        gathered = [torch.zeros_like(copy_rates) for _ in range(world)]
        dist.all_gather(gathered, copy_rates)
    else:
        gathered = [copy_rates]
    numa_nodes = [numa.get("numa_node")]
    if distributed:
        numa_nodes = [None] * world
        dist.all_gather_object(numa_nodes, numa.get("numa_node"))

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
        (gather_ms,) = rank_max(g0.elapsed_time(g1) / 5)
        del full

    # ---------------------------------------------------------------- the drop-in default precision
    value_3x = None
    if extras and args.precision == "tf32":
        step3 = make_step(wl.op, "3xtf32", args.variant)
        for _ in range(3):
            step3(*inputs)
        barrier()
        ms3 = time_steps(lambda: step3(*inputs), max(10, min(steps, 30)), flush)
        (ms3_max,) = rank_max(statistics.median(ms3))
        value_3x = {"value": world * wl.flops / (ms3_max * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms3_max,
                    "note": "precision the drop-in call uses when set_tf32_enabled was never called "
                            "(the reference's default, triturus/utils.py:9); same FLOP count, three MMAs per step"}  # fmt: skip
        tb.check_status()

    # ---------------------------------------------------------------- Triton reference on the same tensors
    triton_ref = None
    if extras and world == 1 and args.triton_ref != "none":
        triton_ref = {wl.name: triton_reference_times(wl, inputs, 20, flush)}

    del host_inputs, host_out, inputs, out
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- strong scaling of the largest configuration
    strong = None
    if extras:
        c5 = WORKLOADS["cfg5"]
        lo, hi = shard_bounds(c5.dims["R"], rank, world)
        xs5 = strong_cfg5_inputs(lo, hi, dev)
        mine = c5.with_batch(hi - lo)
        step5 = make_step("lt2exp", args.precision, 0)
        for _ in range(3):
            step5(*xs5)
        barrier()
        ms5 = time_steps(lambda: step5(*xs5), 20, None)
        barrier()
        (ms5_max,) = rank_max(statistics.median(ms5))
        tb.check_status()
        code = plan_code(mine, args.precision, 0)
        bn, mt = (code % 10000) // 10, code % 10
        rows = 128 * (2 if mt in (2, 4) else 1)
        cols = 256 if (bn == 256 or mt == 5) else 128
        tiles = (hi - lo) * -(-c5.dims["S"] // rows) * -(-c5.dims["K"] // cols)
        strong = {"workload": workload_string(c5), "scaling": "strong", "sharding": f"batch r, {hi - lo} of 64 entries per GPU",
                  "ms_per_step": ms5_max, "value": c5.flops / (ms5_max * 1e-3) / 1e12, "unit": "TFLOP/s",
                  "plan": code, "tiles_per_rank": tiles, "waves_of_tiles": tiles / SM_COUNT,
                  "launches_per_step": launches_per_step(mine, args.precision, 0),
                  "timing": "CUDA events per step, median of 20 after 3 warm-up, max over ranks; inputs resident"}  # fmt: skip
        if args.triton_ref == "all" and world == 1 and triton_ref is not None:
            sample = c5.with_batch(4)
            triton_ref["cfg5 (R=4 of 64)"] = triton_reference_times(sample, [t[:4].contiguous() for t in xs5], 5, None)
        del xs5
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- the other configurations, one GPU
    configs = None
    cublas = None
    peaks = load_peaks()
    if extras and world == 1:
        configs = {}
        for name in ("cfg1", "cfg3", "cfg4"):
            w2 = WORKLOADS[name]
            xs = [t.to(dev) for t in make_inputs(w2, seed=0)]
            st = make_step(w2.op, args.precision, 0)
            fl = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if w2.bytes < 2 * 126e6 else None
            for _ in range(5):
                st(*xs)
            torch.cuda.synchronize()
            q = quantiles(time_steps(lambda: st(*xs), 30, fl))
            r2 = roofline_of(w2, q["p50"], peaks, clocks)
            configs[name] = {"workload": workload_string(w2), "ms": q, "TFLOP/s": w2.flops / (q["p50"] * 1e-3) / 1e12,
                             "roofline": {k: r2[k] for k in r2 if k != "peak_source"}, "plan": plan_code(w2, args.precision, 0),
                             "l2_flushed_between_steps": fl is not None}  # fmt: skip
            del xs, fl
            torch.cuda.empty_cache()
        if strong is not None:
            r5 = roofline_of(WORKLOADS["cfg5"], strong["ms_per_step"], peaks, clocks)
            configs["cfg5"] = {"workload": strong["workload"], "ms": {"p50": strong["ms_per_step"]}, "TFLOP/s": strong["value"],
                               "roofline": {k: r5[k] for k in r5 if k != "peak_source"}, "plan": strong["plan"]}  # fmt: skip
        tb.check_status()
        cublas = cublas_tf32_tflops(dev)

    if rank == 0:
        roof = roofline_of(wl, ms_per_step, peaks, clocks)
        roof["traffic"] = None if custom_dims else NCU_TRAFFIC_BYTES.get((wl.name, args.precision))
        roof["step_ms"] = ms_per_step
        roof["kernels_per_step"] = n_launch
        roof["kernel"] = ("lt2exp_kernel" if wl.op == "lt2exp" else
                          "lm2exp chain link (stabiliser supplied, column maxima returned)" if args.chain else
                          ("colmax_kernel + lm2exp_pair_kernel / lm2exp_kernel" if stab == 1 else
                           "lm2exp_tspair_kernel with the optimistic stabiliser (+ the conditional launch of the same kernel "
                           "with an exact max pass, which returns at once)" if stab == 0 else
                           "lm2exp_kernel, max pass over the first k-block of each slab (+ the conditional launch of the "
                           "full pass, which returns at once)" if stab == 3 else
                           "colmax_kernel over the first 32 rows + lm2exp_pair_kernel (+ two conditional launches of "
                           "the exact passes, which return at once)" if stab == 4
                           else "lm2exp_kernel (fused max pass)"))
        if kernel_ms is not None:
            dom = roofline_of(wl, kernel_ms, peaks, clocks)
            roof["dominant_kernel_ms"] = kernel_ms
            roof["prepass_ms"] = prepass_ms
            roof["frac_dominant_kernel"] = dom["frac"]
            roof["dominant_kernel_note"] = ("contraction kernel timed by itself (column maxima supplied, single launch); "
                                            "frac and achieved are the whole step")
        if cublas is not None and wl.name in TENSOR_BOUND:
            roof["frac_of_cublas_tf32"] = roof["achieved"] / cublas["bmm_32x1024x1024x1024"]

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
                "workload": workload_string(wl, custom_dims),
                "precision": args.precision,
                "variant": args.variant,
                "plan": plan_code(wl, args.precision, args.variant),
                **({"chain": "inner link: b_colmax supplied, out_colmax returned"} if args.chain else {}),
                "sharding": f"batch r, one full batch per GPU x {world}",
                "l2": (f"operands + result = {wl.bytes / 1e6:.0f} MB per step, larger than the 126 MB L2"
                       if flush is None else
                       f"operands + result = {wl.bytes / 1e6:.0f} MB per step fit in the 126 MB L2: "
                       "a 256 MB buffer is written between timed steps"),
            },
            "step_ms_quantiles": quantiles(per_step_ms + more),
            "roofline": roof,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "per_rank": {"h2d_gbs_all_ranks_copying": [float(g[0]) for g in gathered],
                                 "e2e_ms": [float(g[1]) for g in gathered], "numa_node": numa_nodes}},  # fmt: skip
            "gpu_launches": n_launch * steps,
            "clocks": clocks,
            "wall_s": t_wall,
            "host_binding": numa,
        }
        if value_3x is not None:
            line["value_3xtf32"] = value_3x
        if strong is not None:
            line["strong_cfg5"] = strong
        if configs is not None:
            line["configs"] = configs
        if cublas is not None:
            line["tf32_cublas_tflops"] = cublas
        if triton_ref is not None:
            line["triton_ref"] = triton_ref
        if gather_ms is not None:
            line["all_gather_ms"] = gather_ms
        if world == 1 and not args.no_cpu_baseline:
            os.sched_setaffinity(0, all_cores)  # the CPU baseline uses every core of the box again
            base = cpu_reference_time(wl, reps=5 if wl.name != "cfg5" else 1)
            base.pop("ms")
            line["cpu_baseline"] = base
            if extras:
                try:
                    jit = cpu_reference_time(wl, reps=3 if wl.name != "cfg5" else 1, jit=True)
                    jit.pop("ms")
                    line["cpu_baseline_jit"] = jit
                except Exception as exc:  # noqa: BLE001
                    line["cpu_baseline_jit"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
        print(json.dumps(line), flush=True)

    if distributed:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

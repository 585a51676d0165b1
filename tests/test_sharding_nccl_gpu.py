"""GPU, two ranks on two devices, NCCL: the sharded runs of both ops with the CUDA kernels against the same call
on one device.  Batch sharding moves whole batch entries, so the gathered result is bit for bit the single-device
one; column sharding changes the tiling of k, so it is compared at the tolerance of the precision.  Skipped on a
machine with fewer than two GPUs.  No kernel of this library reads a peer's memory: the only traffic between the
ranks is NCCL's all-gather of the results."""

import os
import socket
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ATOL

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]  # fmt: skip


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, failures):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=timedelta(seconds=120),
                            device_id=torch.device("cuda", rank))  # fmt: skip
    try:
        import triturus_b200 as tb
        from triturus_b200.sharding import run_sharded, shard_bounds

        g = torch.Generator().manual_seed(0)
        R = 5  # ragged over two ranks
        a = torch.rand(R, 300, 96, generator=g).cuda()
        b = (torch.randn(R, 96, 520, generator=g) * 5.0).cuda()
        b[R - 1, :, 7] = float("-inf")
        w = torch.rand(R, 70, 16, 24, generator=g).cuda()
        xa = (torch.randn(R, 16, 520, generator=g) * 3.0).cuda()
        xb = (torch.randn(R, 24, 520, generator=g) * 3.0).cuda()
        for precision in ("tf32", "3xtf32"):
            # explicit tiles: the automatic choice looks at the batch size, and another tile is another summation order
            lm = lambda a_, b_: tb.lm2exp(a_, b_, precision=precision, variant=101281)  # noqa: E731
            lt = lambda w_, a_, b_: tb.lt2exp(w_, a_, b_, precision=precision, variant=11281)  # noqa: E731
            full_lm, full_lt = lm(a, b), lt(w, xa, xb)
            for name, op, xs, full in (("lm2exp", lm, (a, b), full_lm), ("lt2exp", lt, (w, xa, xb), full_lt)):
                got = run_sharded(op, xs, gather=True, axis="batch")
                if not torch.equal(got, full):
                    failures.append(f"rank {rank} {precision}: batch-gathered {name} differs from one device")
                mine = run_sharded(op, xs, gather=False, axis="batch")
                lo, hi = shard_bounds(R, rank, world)
                if not torch.equal(mine, full[lo:hi]):
                    failures.append(f"rank {rank} {precision}: local batch shard of {name} differs")
                cols = run_sharded(op, xs, gather=True, axis="columns")
                fin = torch.isfinite(full)
                if cols.shape != full.shape or not torch.equal(torch.isinf(cols), torch.isinf(full)) or \
                        (cols - full)[fin].abs().max().item() > 2 * ATOL[precision]:
                    failures.append(f"rank {rank} {precision}: column-gathered {name} differs")
            tb.check_status()
    except Exception as exc:  # noqa: BLE001
        failures.append(f"rank {rank}: {type(exc).__name__}: {exc}")
    finally:
        dist.destroy_process_group()


def test_two_gpus_sharded_runs_match_one_device():
    world = 2
    with mp.Manager() as mgr:
        failures = mgr.list()
        mp.spawn(_worker, args=(world, _free_port(), failures), nprocs=world, join=True)
        assert list(failures) == []

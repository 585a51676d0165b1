"""CPU, world_size 2, gloo: the batch-sharding host logic (bounds, slicing, ragged all-gather).  The op
applied to each shard is the CPU oracle, standing in for the CUDA kernels, because the logic under test is
the partitioning and the gather, not the arithmetic."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from triturus_b200.sharding import shard_bounds


def test_shard_bounds_cover_the_batch():
    for batch in (0, 1, 5, 8, 32, 33):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            for (lo0, hi0), (lo1, hi1) in zip(spans, spans[1:]):
                assert hi0 == lo1 and hi0 - lo0 >= hi1 - lo1 >= 0
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def test_column_bounds_cover_the_columns_on_aligned_cuts():
    from triturus_b200.sharding import column_bounds

    for columns in (0, 3, 8, 100, 256, 8192, 530):
        for world in (1, 2, 3, 8):
            spans = [column_bounds(columns, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == columns
            for (lo0, hi0), (lo1, hi1) in zip(spans, spans[1:]):
                assert hi0 == lo1
            if columns % 4 == 0:
                assert all(lo % 4 == 0 for lo, _ in spans)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, batch: int, failures):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.logspace_oracle import lm2exp_fp32, lt2exp_fp32
        from triturus_b200.sharding import run_sharded, shard_batch

        g = torch.Generator().manual_seed(0)
        a = torch.rand(batch, 9, 7, generator=g)
        b = torch.randn(batch, 7, 11, generator=g)
        w = torch.rand(batch, 5, 3, 7, generator=g)
        x = torch.randn(batch, 3, 11, generator=g)
        full_lm = lm2exp_fp32(a, b)
        full_lt = lt2exp_fp32(w, x, b)
        got = run_sharded(lm2exp_fp32, (a, b), gather=True, axis="batch")
        if not torch.equal(got, full_lm):
            failures.append(f"rank {rank}: gathered lm2exp differs")
        got = run_sharded(lt2exp_fp32, (w, x, b), gather=True, axis="batch")
        if not torch.equal(got, full_lt):
            failures.append(f"rank {rank}: gathered lt2exp differs")
        mine = run_sharded(lm2exp_fp32, (a, b), gather=False, axis="batch")
        lo, hi = shard_bounds(batch, rank, world)
        if not torch.equal(mine, full_lm[lo:hi]):
            failures.append(f"rank {rank}: local shard differs")
        sa, sb = shard_batch((a, b), rank, world)
        if sa.data_ptr() != a[lo:hi].data_ptr() or sb.shape[0] != hi - lo:
            failures.append(f"rank {rank}: shard_batch is not a view of the block")
        # column sharding (what axis="auto" picks when the batch has fewer entries than there are ranks)
        from triturus_b200.sharding import column_bounds, shard_columns

        for op, xs, full in ((lm2exp_fp32, (a, b), full_lm), (lt2exp_fp32, (w, x, b), full_lt)):
            got = run_sharded(op, xs, gather=True, axis="columns")
            if got.shape != full.shape or not torch.allclose(got, full, rtol=1e-6, atol=1e-6):
                failures.append(f"rank {rank}: column-gathered {op.__name__} differs")
            mine = run_sharded(op, xs, gather=False, axis="columns")
            klo, khi = column_bounds(b.shape[-1], rank, world)
            if not torch.allclose(mine, full[..., klo:khi], rtol=1e-6, atol=1e-6):
                failures.append(f"rank {rank}: local column shard of {op.__name__} differs")
        auto = run_sharded(lm2exp_fp32, (a, b), gather=False)
        want_cols = batch < world
        if (auto.shape[0] == batch and auto.shape[-1] < b.shape[-1]) != want_cols:
            failures.append(f"rank {rank}: axis=auto picked the wrong axis for batch {batch}")
        sc = shard_columns((w, x, b), rank, world)
        if sc[0].data_ptr() != w.data_ptr() or sc[2].shape[-1] != khi - klo:
            failures.append(f"rank {rank}: shard_columns must replicate w and slice k")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch", [4, 5, 1])
def test_two_rank_sharded_run_matches_single_process(batch):
    world = 2
    with mp.Manager() as mgr:
        failures = mgr.list()
        mp.spawn(_worker, args=(world, _free_port(), batch, failures), nprocs=world, join=True)
        assert list(failures) == []

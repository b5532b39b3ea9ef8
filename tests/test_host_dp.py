"""CPU tests of the data-parallel host logic, with real world_size-2 process groups over gloo:
the flat-bucket sum-allreduce, the non-finite-flag consensus and the loss-scale sawtooth
(crates/loractl-core/src/diffusion_trainer.rs:270-276,1703-1743)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from loractl_b200 import dp
from loractl_b200.optim import (INITIAL_LOSS_SCALE, MAX_LOSS_SCALE, MIN_LOSS_SCALE, SCALE_GROWTH_INTERVAL,
                                DynamicLossScale)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # step 1: finite gradients on both ranks -> mean over ranks, nobody skips
        bucket = torch.arange(10, dtype=torch.float32) * (rank + 1)
        flag = torch.zeros(1, dtype=torch.int32)
        scale = dp.sync_gradients(bucket, flag)
        scaler = DynamicLossScale()
        finite1, warn1 = dp.consensus_step(scaler, flag)
        mean = bucket * scale
        # step 2: only rank 1 saw a non-finite gradient -> BOTH ranks must skip and halve
        bucket2 = torch.ones(10)
        flag2 = torch.tensor([1 if rank == 1 else 0], dtype=torch.int32)
        if rank == 1:
            bucket2[3] = float("inf")
        dp.sync_gradients(bucket2, flag2)
        finite2, warn2 = dp.consensus_step(scaler, flag2)
        # async form returns handles
        b3 = torch.full((4,), float(rank))
        s3, handles = dp.sync_gradients(b3, None, async_op=True)
        for h in handles:
            h.wait()
        out.put((rank, mean.tolist(), scale, finite1, warn1, finite2, warn2, scaler.loss_scale, b3.tolist(), s3))
    finally:
        dist.destroy_process_group()


def test_two_rank_bucket_allreduce_and_skip_consensus():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, mean, scale, finite1, warn1, finite2, warn2, ls, b3, s3 in res:
        assert scale == 0.5 and s3 == 0.5
        assert mean == [1.5 * i for i in range(10)]  # (1 + 2) / 2 * i
        assert finite1 and warn1 is None
        assert not finite2 and "loss scale halved" in warn2  # rank 0 skips too
        assert ls == INITIAL_LOSS_SCALE / 2
        assert b3 == [1.0] * 4


def test_single_process_is_identity():
    b = torch.ones(5)
    assert dp.sync_gradients(b, torch.zeros(1, dtype=torch.int32)) == 1.0
    assert b.tolist() == [1.0] * 5


def test_loss_scale_sawtooth():
    s = DynamicLossScale()
    assert s.loss_scale == INITIAL_LOSS_SCALE
    for _ in range(SCALE_GROWTH_INTERVAL - 1):
        assert s.update(True) is None
    assert s.loss_scale == INITIAL_LOSS_SCALE
    s.update(True)
    assert s.loss_scale == 2 * INITIAL_LOSS_SCALE and s.clean_streak == 0
    for _ in range(3 * SCALE_GROWTH_INTERVAL):
        s.update(True)
    assert s.loss_scale == MAX_LOSS_SCALE  # capped
    msg = s.update(False)
    assert "halved" in msg and s.loss_scale == MAX_LOSS_SCALE / 2 and s.clean_streak == 0
    for _ in range(40):
        s.update(False)
    assert s.loss_scale == MIN_LOSS_SCALE  # floored


@pytest.mark.parametrize("batch,world", [(8, 1), (8, 2), (8, 8), (7, 3), (2, 4)])
def test_shard_range_partitions_the_batch(batch, world):
    spans = [dp.shard_range(batch, r, world) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == batch
    assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
    sizes = [b - a for a, b in spans]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


def _bucket_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # three "blocks" of a flat bucket, reduced from the last block to the first as a reverse
        # sweep would, each slice as soon as it is final
        bucket = torch.arange(12, dtype=torch.float32) * (rank + 1)
        red = dp.BucketReducer(bucket)
        for lo, hi in ((8, 12), (3, 8), (0, 3)):
            red.reduce_slice(lo, hi)
        scale = red.finish()
        flag = torch.tensor([1 if rank == 1 else 0], dtype=torch.int32)
        dp.reduce_flag(flag)
        out.put((rank, bucket.tolist(), scale, int(flag.item())))
    finally:
        dist.destroy_process_group()


def test_two_rank_per_block_buckets_equal_one_flat_allreduce():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_bucket_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    want = [float(i) * 3 for i in range(12)]  # rank 0 contributes i, rank 1 contributes 2 i
    for rank, bucket, scale, flag in res:
        assert bucket == want and scale == 0.5 and flag == 1
    # one rank: nothing to reduce, scale 1
    red = dp.BucketReducer(torch.ones(4))
    red.reduce_slice(0, 4)
    assert red.finish() == 1.0


def test_sweep_reduce_ranges_cover_every_block_once():
    """Blocks per gradient all-reduce of the reverse sweep: whatever the grouping, every block's slice is
    reduced exactly once, each range is due only when its lowest block's backward has been enqueued,
    and grouping all blocks gives the single all-reduce after the sweep."""
    from loractl_b200.dp import sweep_reduce_range

    for n_blocks in (1, 2, 5, 24):
        for every in (1, 2, 4, 5, 24, 100):
            seen = []
            for i in range(n_blocks - 1, -1, -1):
                due = sweep_reduce_range(n_blocks, every, i)
                if due is not None:
                    lo, hi = due
                    assert lo == i and lo <= hi < n_blocks and hi - lo + 1 <= every
                    seen += list(range(lo, hi + 1))
            assert sorted(seen) == list(range(n_blocks)), (n_blocks, every, seen)
    assert sweep_reduce_range(24, 24, 0) == (0, 23)
    assert all(sweep_reduce_range(24, 24, i) is None for i in range(1, 24))
    assert sweep_reduce_range(24, 1, 7) == (7, 7)

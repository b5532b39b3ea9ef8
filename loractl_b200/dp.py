"""Data-parallel exchange of the LoRA path: the only collective is a sum-allreduce of the flat
LoRA-gradient bucket (plus a 1-element max-allreduce of the non-finite flag so every rank takes
the same skip decision).  The reference is single-device (`compute.device` is one ordinal,
crates/loractl-core/src/config.rs:707-710); N replicas here equal one replica with N times the
batch: each rank's loss is a mean over its shard, so gradients are averaged (`1/world`), which
the fused AdamW applies as its `grad_scale`.

The functions take plain tensors and a process group, so the same code runs over NCCL on GPUs
and over gloo on CPU tensors (which is how the host logic is tested without GPUs)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .optim import DynamicLossScale


def world_size(group=None) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def sync_gradients(bucket: torch.Tensor, flag: Optional[torch.Tensor] = None, group=None,
                   async_op: bool = False):
    """Sum-allreduce the flat gradient bucket in place and (if given) max-allreduce the
    non-finite flag.  Returns the scale (`1/world`) that turns the sum into the mean."""
    n = world_size(group)
    handles = []
    if n > 1:
        handles.append(dist.all_reduce(bucket, op=dist.ReduceOp.SUM, group=group, async_op=async_op))
        if flag is not None:
            handles.append(dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group, async_op=async_op))
    if async_op:
        return 1.0 / n, [h for h in handles if h is not None]
    return 1.0 / n


class BucketReducer:
    """Per-block gradient buckets reduced while the reverse sweep is still running.

    The flat gradient buffer holds the adapters in registration order, so the gradients of one
    block are one contiguous slice.  `reduce_slice(lo, hi)` starts a sum-allreduce of that slice as
    soon as the block's backward has been enqueued (NCCL orders it after the kernels already on the
    current stream and runs it on its own stream); `finish()` waits for all of them and reduces the
    non-finite flag.  With one rank everything is a no-op."""

    def __init__(self, bucket: torch.Tensor, group=None):
        self.bucket, self.group, self.handles = bucket, group, []
        self.world = world_size(group)

    def reduce_slice(self, lo: int, hi: int) -> None:
        if self.world > 1 and hi > lo:
            self.handles.append(dist.all_reduce(self.bucket[lo:hi], op=dist.ReduceOp.SUM, group=self.group,
                                                async_op=True))

    def finish(self) -> float:
        """Waits for every slice; returns the scale (`1/world`) that turns the sums into means."""
        for h in self.handles:
            h.wait()
        self.handles = []
        return 1.0 / self.world


def sweep_reduce_range(n_blocks: int, reduce_every: int, i: int):
    """Blocks whose gradients are all-reduced right after block `i`'s backward in a reverse sweep
    (`i` runs from `n_blocks - 1` down to 0) when one all-reduce covers `reduce_every` blocks: `(lo, hi)`
    inclusive, or None when nothing is due yet.  Every block is covered exactly once; the last range
    (at `i == 0`) may be shorter."""
    reduce_every = max(int(reduce_every), 1)
    done = n_blocks - i  # blocks whose gradients are final, counted from the top
    if done % reduce_every != 0 and i != 0:
        return None
    return i, min(i + (done - 1) % reduce_every, n_blocks - 1)


def reduce_flag(flag: torch.Tensor, group=None) -> None:
    """Max-allreduce of the 1-element non-finite flag, so that every rank takes the same decision."""
    if world_size(group) > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)


def consensus_step(scaler: DynamicLossScale, flag: torch.Tensor) -> Tuple[bool, Optional[str]]:
    """Reads the (already all-reduced) flag — the one host synchronisation per step, where the
    reference reads its |g| sum (crates/loractl-core/src/diffusion_trainer.rs:1724) — and
    advances the loss-scale sawtooth.  Every rank sees the same flag, so every rank skips or
    steps together and the replicas never diverge."""
    finite = int(flag.item()) == 0
    return finite, scaler.update(finite)


def shard_range(global_batch: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous sample shard of `rank`: sizes differ by at most one, earlier ranks take the
    extra sample."""
    base, rem = divmod(global_batch, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)

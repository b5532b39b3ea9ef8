"""Block-level gradient checkpointing — the mirror of crates/loractl-core/src/block_ckpt.rs.

`checkpointed_step` reproduces the reference's three phases (block_ckpt.rs:103-207):
  1. capture: run the trunk without a graph, storing each block's input;
  2. head graph: loss from the final activation, backward to get dL/dx_final;
  3. reverse sweep: per block, lift its stored input as a fresh leaf, replay the block
     forward (the SAME LoRA-linear kernels: one more forward per site), seed the backward
     with the incoming gradient, collect adapter gradients, pass dL/dx to the block below.
Peak activation memory is one block's interior.  It requires deterministic kernels (the replayed
forward must equal the captured one) and no dropout on the adapters
(crates/loractl-core/src/diffusion_trainer.rs:342-348)."""
from __future__ import annotations

from typing import Callable, Iterable, List, Optional, Sequence, Tuple

import torch


def checkpointed_step(blocks: Sequence[Callable[[torch.Tensor], torch.Tensor]], x0: torch.Tensor,
                      head_loss: Callable[[torch.Tensor], torch.Tensor], params: Iterable[torch.nn.Parameter],
                      loss_scale: float = 1.0, keep_existing_grads: bool = False,
                      after_block: Optional[Callable[[int], None]] = None) -> Tuple[float, List[torch.Tensor]]:
    """One training step's loss and gradients with block-checkpoint recompute.

    blocks     the trunk, each `block(x) -> x` (adapters are closed over, as the reference passes
               the per-block adapter subset into the replayed block, block_ckpt.rs:128-143,176-184)
    x0         the trunk's input (output of the pre-trunk stage)
    head_loss  final activation -> scalar loss (`LastLayer` + MSE in the reference, :145-156)
    params     the adapter parameters whose gradients are wanted
    after_block  called with the block index once that block's backward has been enqueued: its adapter
               gradients are final from then on (a data-parallel trainer starts their all-reduce
               here, so that it overlaps the replay of the blocks below)
    Returns `(loss, grads)` with `grads[i] = d(loss * loss_scale) / d params[i]`, the same
    quantities `(loss * loss_scale).backward()` of the monolithic step produces.
    """
    params = list(params)
    if not keep_existing_grads:  # with a flat gradient bucket the (zeroed) .grad views are kept and added into
        for p in params:
            p.grad = None
    # Phase 1 — capture (no graph)
    block_inputs: List[torch.Tensor] = []
    with torch.no_grad():
        x = x0
        for blk in blocks:
            block_inputs.append(x)
            x = blk(x)
    # Phase 2 — head graph
    x_final = x.detach().requires_grad_(True)
    loss = head_loss(x_final)
    (loss * loss_scale).backward()
    grad_x = x_final.grad
    loss_dev = loss.detach()  # read back after the sweep is enqueued: a host read here would drain the GPU
    # Phase 3 — reverse sweep with per-block replay
    for i in range(len(blocks) - 1, -1, -1):
        x2 = block_inputs[i].detach().requires_grad_(True)
        out = blocks[i](x2)
        out.backward(gradient=grad_x)  # the reference seeds via (out * g).sum().backward(): same VJP
        grad_x = x2.grad
        block_inputs[i] = None  # release as the sweep passes
        if after_block is not None:
            after_block(i)
    grads = [p.grad if p.grad is not None else torch.zeros_like(p) for p in params]
    return float(loss_dev), grads

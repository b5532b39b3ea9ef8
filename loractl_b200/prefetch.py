"""bf16 weight copies one block ahead of the compute.

The tensor-regime calls rebuild a bf16 image of the frozen weight in their workspace on every call
(the reference rebuilds an f32 one: crates/loractl-core/src/quant.rs:232-233,250-251).  Under block
checkpointing (crates/loractl-core/src/block_ckpt.rs:103-207) a step visits the blocks in a known
order — 0..L-1 without a graph, then L-1..0 with replay and backward — so the image of the NEXT
block's weights can be built on a side stream while the current block computes, into one of two
arenas that each hold one block's copies (`QuantWeight.attach_bf16_copy`).  The calls of the block
then read the copy in place — the forward as a K-major operand, the backward the same bytes as an
MN-major operand — and run no dequantisation pass; a block's replay and its backward share one
copy.  Memory: two blocks' bf16 weights instead of the whole stack's.

Ordering: a slot's previous occupant is always two blocks away in the sweep, so all of its work is
already enqueued on the compute stream when the refill is requested; the side stream waits for an
event recorded on the compute stream at that moment, and the compute stream waits for the refill's
event before the block that needs it."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .quant import QuantWeight


class BlockWeightPrefetcher:
    def __init__(self, block_weights: Sequence[Sequence[QuantWeight]], device):
        self.weights: List[List[QuantWeight]] = [list(ws) for ws in block_weights]
        self.device = torch.device(device)
        align = 128  # elements: every copy starts on a 256-byte boundary
        self.offsets: List[List[int]] = []
        need = 0
        for ws in self.weights:
            offs, off = [], 0
            for w in ws:
                offs.append(off)
                off += -(-(w.d_out * w.d_in) // align) * align
            self.offsets.append(offs)
            need = max(need, off)
        self.arenas = [torch.empty(max(need, align), dtype=torch.bfloat16, device=self.device) for _ in range(2)]
        self.stream = torch.cuda.Stream(device=self.device)
        self.occupant: List[Optional[int]] = [None, None]
        self.ready: Dict[int, torch.cuda.Event] = {}
        self.fills = 0  # refills issued, for tests and accounting

    @staticmethod
    def slot(i: int) -> int:
        return i & 1

    def fill(self, i: int, stream) -> None:
        """Block i's copies rebuilt into its slot on `stream`, with no ordering of its own (the caller
        orders `stream` against the readers of the slot's previous content and of the new one)."""
        s = self.slot(i)
        old = self.occupant[s]
        if old is not None and old != i:
            for w in self.weights[old]:
                w.detach_bf16_copy()
            self.ready.pop(old, None)
        arena = self.arenas[s]
        with torch.cuda.stream(stream):
            for w, off in zip(self.weights[i], self.offsets[i]):
                w.attach_bf16_copy(arena[off:off + w.d_out * w.d_in])
        self.occupant[s] = i
        self.fills += 1

    def prefetch(self, i: int) -> None:
        """Starts building block i's copies on the side stream unless they are in place already."""
        if i < 0 or i >= len(self.weights) or self.occupant[self.slot(i)] == i:
            return
        s = self.slot(i)
        old = self.occupant[s]
        if old is not None:  # host-side state only: launches already enqueued keep their pointers
            for w in self.weights[old]:
                w.detach_bf16_copy()
            self.ready.pop(old, None)
        main = torch.cuda.current_stream(self.device)
        fence = torch.cuda.Event()
        fence.record(main)  # everything that read the slot's previous content is enqueued before this
        self.stream.wait_event(fence)
        arena = self.arenas[s]
        with torch.cuda.stream(self.stream):
            for w, off in zip(self.weights[i], self.offsets[i]):
                w.attach_bf16_copy(arena[off:off + w.d_out * w.d_in])
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.occupant[s] = i
        self.ready[i] = ev
        self.fills += 1

    def acquire(self, i: int) -> None:
        """Block i is about to run on the current stream: its copies must be complete before it reads them."""
        self.prefetch(i)
        ev = self.ready.get(i)
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)

    def release_all(self) -> None:
        for s, occ in enumerate(self.occupant):
            if occ is not None:
                for w in self.weights[occ]:
                    w.detach_bf16_copy()
            self.occupant[s] = None
        self.ready.clear()

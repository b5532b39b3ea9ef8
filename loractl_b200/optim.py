"""Step glue on flat LoRA buffers — the mirror of the optimizer section of
crates/loractl-core/src/diffusion_trainer.rs:1564-1566,1703-1743 (AdamW over the adapter set,
finite-gradient guard, dynamic loss-scale sawtooth).

Every adapter's `lora_a` / `lora_b` is re-homed as a view into ONE flat f32 parameter buffer with
a parallel flat gradient buffer.  The LoRA-linear backward writes dA/dB straight into the gradient
views, NCCL all-reduces the one buffer, the finite check is one kernel and AdamW is one kernel.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import _lib as L
from .adapters import LoraAdapters

# crates/loractl-core/src/diffusion_trainer.rs:270-276
INITIAL_LOSS_SCALE = 16384.0
MAX_LOSS_SCALE = 65536.0
MIN_LOSS_SCALE = 1.0
SCALE_GROWTH_INTERVAL = 50


class DynamicLossScale:
    """The sawtooth of diffusion_trainer.rs:1727-1743: a clean step grows the streak and after
    `SCALE_GROWTH_INTERVAL` clean steps the scale doubles (capped); a non-finite step resets the
    streak and halves the scale (floored).  Pure host state, restored on resume like the
    reference's sidecar (`crates/loractl-core/src/resume.rs:68-96`)."""

    def __init__(self, initial: float = INITIAL_LOSS_SCALE):
        self.loss_scale = float(initial)
        self.clean_streak = 0

    def update(self, grads_finite: bool) -> Optional[str]:
        """Returns the reference's warning text when the step was skipped, else None."""
        if grads_finite:
            self.clean_streak += 1
            if self.clean_streak >= SCALE_GROWTH_INTERVAL and self.loss_scale < MAX_LOSS_SCALE:
                self.loss_scale = min(self.loss_scale * 2.0, MAX_LOSS_SCALE)
                self.clean_streak = 0
            return None
        self.clean_streak = 0
        self.loss_scale = max(self.loss_scale / 2.0, MIN_LOSS_SCALE)
        return f"non-finite gradients — update skipped, loss scale halved to {self.loss_scale:g}"


class FlatAdapters:
    """Flat parameter / gradient / moment buffers over a `LoraAdapters` set.

    Layout: for each delta in registration order, `lora_a` ([d_in, r], row-major) then `lora_b`
    ([r, d_out]); every segment starts on a 64-float boundary so that kernels may use 16-byte
    accesses.  After construction each `delta.lora_a` / `delta.lora_b` IS a view of `params`, and
    `.grad` of each is a view of `grads`."""

    ALIGN = 64

    def __init__(self, adapters: LoraAdapters, device=None):
        self.adapters = adapters
        params = [p for d in adapters.deltas for p in (d.lora_a, d.lora_b)]
        device = device if device is not None else (params[0].device if params else torch.device("cpu"))
        self.offsets: List[int] = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        self.numel = off
        self.params = torch.zeros(off, dtype=torch.float32, device=device)
        self.grads = torch.zeros(off, dtype=torch.float32, device=device)
        self.exp_avg = torch.zeros(off, dtype=torch.float32, device=device)
        self.exp_avg_sq = torch.zeros(off, dtype=torch.float32, device=device)
        self.flag = torch.zeros(1, dtype=torch.int32, device=device)
        for p, o in zip(params, self.offsets):
            seg = self.params[o:o + p.numel()].view(p.shape)
            seg.copy_(p.detach().to(device))
            p.data = seg
            p.grad = self.grads[o:o + p.numel()].view(p.shape)
        self._params = params
        self.param_epoch = [0]  # shared with every delta: bumped when a kernel rewrites `params`
        for i, d in enumerate(adapters.deltas):
            d.param_epoch = self.param_epoch
            d.bucket_grads = (params[2 * i].grad, params[2 * i + 1].grad)

    def refresh_mirrors(self) -> None:
        """Rebuilds the bf16 operand mirror of every adapter whose factors changed since it was built,
        with one launch per 24 adapters (after `AdamW.step`, instead of one launch per site at its
        first use in the next forward)."""
        from . import quant as Q

        if not self.params.is_cuda:
            return
        jobs, stale = [], []
        for d in self.adapters.deltas:
            key = d._mirror_state()
            if d._mirror is not None and d._mirror_key == key:
                continue
            if d._mirror is None:
                d._mirror = Q.lora_mirror_alloc(d.lora_a, d.lora_b)
            jobs.append((d.lora_a.detach(), d.lora_b.detach(), d._mirror))
            stale.append((d, key))
        Q.lora_mirror_batch(jobs)
        for d, key in stale:
            d._mirror_key = key

    def grad_views(self, index: int):
        """(dA view, dB view) of delta `index` — pass them to `lq_linear_bwd` as outputs."""
        a, b = self._params[2 * index], self._params[2 * index + 1]
        return a.grad, b.grad

    def zero_grad(self) -> None:
        self.grads.zero_()
        for p, o in zip(self._params, self.offsets):  # autograd may have replaced .grad
            if p.grad is None or p.grad.data_ptr() != self.grads.data_ptr() + 4 * o:
                p.grad = self.grads[o:o + p.numel()].view(p.shape)

    def gather_autograd_grads(self, only: Optional[tuple] = None) -> None:
        """If autograd accumulated into separate `.grad` tensors, fold them back into the bucket
        (`only` = (lo, hi): just the parameters whose segment starts inside that slice)."""
        import bisect

        lo = 0 if only is None else bisect.bisect_left(self.offsets, only[0])
        hi = len(self.offsets) if only is None else bisect.bisect_left(self.offsets, only[1])
        for p, o in zip(self._params[lo:hi], self.offsets[lo:hi]):
            if p.grad is not None and p.grad.data_ptr() != self.grads.data_ptr() + 4 * o:
                self.grads[o:o + p.numel()].view(p.shape).copy_(p.grad)
                p.grad = self.grads[o:o + p.numel()].view(p.shape)


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def nonfinite_flag(grads: torch.Tensor, flag: torch.Tensor) -> None:
    """One-kernel finite check over the flat gradient buffer (diffusion_trainer.rs:1708-1725):
    `flag[0]` becomes 1 iff some gradient is NaN/Inf.  No host synchronisation."""
    if not grads.is_cuda:
        raise RuntimeError("the b200 backend has no CPU path")
    with torch.cuda.device(grads.device):
        L.check(L.lib().lq_grad_nonfinite_flag(grads.data_ptr(), grads.numel(), flag.data_ptr(), _stream(grads)))


class AdamW:
    """burn `AdamWConfig::new().with_weight_decay(wd)` (diffusion_trainer.rs:1564-1566) over a
    `FlatAdapters`: defaults beta1 0.9, beta2 0.999, epsilon 1e-5 (burn-optim 0.21), decoupled
    decay.  `step()` is one kernel; with `skip_flag` it skips itself on the device."""

    def __init__(self, flat: FlatAdapters, weight_decay: float = 1e-4, beta1: float = 0.9, beta2: float = 0.999,
                 eps: float = 1e-5):
        self.flat, self.weight_decay, self.beta1, self.beta2, self.eps = flat, weight_decay, beta1, beta2, eps
        self.steps = 0

    def step(self, lr: float, grad_scale: float = 1.0, skip_flag: Optional[torch.Tensor] = None,
             count: bool = True) -> None:
        f = self.flat
        if not f.params.is_cuda:
            raise RuntimeError("the b200 backend has no CPU path")
        if count:
            self.steps += 1
        with torch.cuda.device(f.params.device):
            L.check(L.lib().lq_adamw_step(
                f.params.data_ptr(), f.grads.data_ptr(), f.exp_avg.data_ptr(), f.exp_avg_sq.data_ptr(), f.numel,
                float(lr), self.beta1, self.beta2, self.eps, float(self.weight_decay), max(self.steps, 1),
                float(grad_scale), skip_flag.data_ptr() if skip_flag is not None else None, _stream(f.params)))
        f.param_epoch[0] += 1  # the kernel wrote through raw pointers: bf16 operand mirrors are stale

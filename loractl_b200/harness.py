"""Callers of the hot path, as PyTorch harnesses: a double-stream MMDiT block whose every linear
is a LoRA'd quantized site, a stack of such blocks, and one data-parallel training step built
from the pieces this package provides (site -> fused LoRA-linear kernels, block-checkpoint
recompute, flat gradient bucket, bucket all-reduce, fused finite check and AdamW).

The block has the shape of the benchmark's double-stream MMDiT block — hidden 3072, 24 heads x 128, MLP 12288;
per stream a joint-qkv 3072 -> 9216, out-projection 3072 -> 3072, MLP up 3072 -> 12288 / down
12288 -> 3072 and an adaLN modulation 3072 -> 18432 on the conditioning vector — which is a
synthetic composition: the reference's own denoiser is the single-stream Krea-2 DiT
(crates/loractl-core/src/mmdit.rs:540-870), whose injectable sites this mirrors only in kind
(`site()` at mmdit.rs:526-536 around each projection).  The modulated layer norms and the gated
residuals are this package's fused element-wise kernels (`block_ops`); attention and GELU are
plain PyTorch ops — the callers either side of the path.

The step mirrors crates/loractl-core/src/diffusion_trainer.rs:1599-1743 with
`compute.grad_checkpointing` on: flow-matching inputs (crates/loractl-core/src/flow.rs:50-66),
block-checkpointed forward/backward (block_ckpt.rs:103-207), finite-gradient guard with the
dynamic loss scale, AdamW over the adapter set.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from . import dp
from .adapters import LoraAdapters, LoraConfig, LoraSite, TargetSpec, build_adapters
from .block_ckpt import checkpointed_step
from .block_ops import gated_residual, modulated_layer_norm
from .linear import BaseLinear, QuantLinear, site, site_group
from .prefetch import BlockWeightPrefetcher
from .optim import AdamW, DynamicLossScale, FlatAdapters, nonfinite_flag
from .quant import quantize_linear_weight


@dataclass
class BlockConfig:
    hidden: int = 3072
    heads: int = 24
    mlp: int = 12288
    img_tokens: int = 4096
    txt_tokens: int = 512
    quant_bits: int = 4
    quant_block: int = 64


def _quant_site(d_in: int, d_out: int, cfg: BlockConfig, gen: torch.Generator, device) -> BaseLinear:
    """A frozen base linear with N(0, 0.02) weights, quantized on the device (the random-init
    stand-in for `Mmdit::into_quantized`, crates/loractl-core/src/mmdit.rs:1122-1158)."""
    w = torch.randn((d_out, d_in), generator=gen, device=device, dtype=torch.float32) * 0.02
    return BaseLinear.quant(QuantLinear(quantize_linear_weight(w, cfg.quant_bits, cfg.quant_block)))


class _SplitStreams(torch.autograd.Function):
    """`[b, img + txt, h]` -> contiguous `[b, img, h]`, `[b, txt, h]`, once per tensor: with b > 1 the
    plain slices are non-contiguous and every fused op behind them made its own strided copy, every
    slice backward its own zero-filled full-size gradient.  The backward is one concatenation."""

    @staticmethod
    def forward(ctx, x, li):
        return x[:, :li].contiguous(), x[:, li:].contiguous()

    @staticmethod
    def backward(ctx, g_img, g_txt):
        return torch.cat([g_img, g_txt], dim=1), None


def split_streams(x: torch.Tensor, li: int):
    """(image part, text part) of `[b, img + txt, h]` along the token axis, each contiguous."""
    if x.shape[0] == 1:  # the slices of a single sample are contiguous views already
        return x[:, :li], x[:, li:]
    return _SplitStreams.apply(x, li)


class DoubleStreamBlock(nn.Module):
    """One double-stream block; the block state is the concatenation [img tokens | txt tokens]
    along the sequence axis so that block-checkpointing sees a single tensor."""

    STREAMS = ("img", "txt")
    LINEARS = ("mod", "qkv", "out", "up", "down")
    _SIDE_STREAMS: dict = {}

    def __init__(self, index: int, cfg: BlockConfig, gen: torch.Generator, device):
        super().__init__()
        self.index, self.cfg = index, cfg
        h, m = cfg.hidden, cfg.mlp
        dims = {"mod": (h, 6 * h), "qkv": (h, 3 * h), "out": (h, h), "up": (h, m), "down": (m, h)}
        self.bases = nn.ModuleDict({f"{s}_{n}": _quant_site(*dims[n], cfg, gen, device)
                                    for s in self.STREAMS for n in self.LINEARS})
        self.adapters: Optional[LoraAdapters] = None
        self.cond: Optional[torch.Tensor] = None  # [b, hidden] conditioning, set per step
        self.two_cuda_streams = False

    def sites(self) -> List[LoraSite]:
        return [LoraSite(self.path(s, n), self.bases[f"{s}_{n}"].d_in, self.bases[f"{s}_{n}"].d_out)
                for s in self.STREAMS for n in self.LINEARS]

    def path(self, stream: str, name: str) -> str:
        return f"blocks.{self.index}.{stream}.{name}"

    def _lin(self, stream: str, name: str, x: torch.Tensor) -> torch.Tensor:
        return site(self.adapters, self.path(stream, name), self.bases[f"{stream}_{name}"], x)

    def _on_two_streams(self, fn) -> dict:
        """`fn(s)` for both token streams.  With `two_cuda_streams` the text stream's chain runs on a second
        CUDA stream beside the image stream's (forked from and joined back into the current stream, so
        a stream capture records two parallel branches): its short kernels — 512 tokens per sample
        against 4096 — fill the gaps of the long ones instead of queueing behind them."""
        if not self.two_cuda_streams:
            return {s: fn(s) for s in self.STREAMS}
        cur = torch.cuda.current_stream()
        key = (cur.device.index, cur.cuda_stream)  # one second stream per (device, calling stream), shared by all blocks
        side = self._SIDE_STREAMS.get(key)
        if side is None:
            side = self._SIDE_STREAMS[key] = torch.cuda.Stream(device=cur.device)
        side.wait_stream(cur)
        out = {}
        with torch.cuda.stream(side):
            out["txt"] = fn("txt")
        out["img"] = fn("img")
        cur.wait_stream(side)
        return out

    def forward(self, state: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        b, _, h = state.shape
        li = cfg.img_tokens
        xs = dict(zip(self.STREAMS, split_streams(state, li)))
        cond = F.silu(self.cond.to(state.dtype))
        # both streams' modulation projections read the same conditioning vector: one grouped call
        mod_out = site_group(self.adapters, [(self.path(s, "mod"), self.bases[f"{s}_mod"]) for s in self.STREAMS], cond)
        mods = {s: mo.unsqueeze(1).chunk(6, dim=-1) for s, mo in zip(self.STREAMS, mod_out)}

        def to_qkv(s):
            xn = modulated_layer_norm(xs[s], mods[s][0], mods[s][1])  # LN(x) * (1 + scale) + shift, one kernel
            return self._lin(s, "qkv", xn).view(b, -1, 3, cfg.heads, h // cfg.heads)

        qkvs = self._on_two_streams(to_qkv)
        qkv = torch.cat([qkvs["img"], qkvs["txt"]], dim=1)  # joint attention over both streams
        q, k, v = (t.transpose(1, 2) for t in qkv.unbind(2))
        att = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, -1, h)
        atts = dict(zip(self.STREAMS, split_streams(att, li)))

        def after_attention(s):
            _, _, gate1, shift2, scale2, gate2 = mods[s]
            x = gated_residual(xs[s], gate1, self._lin(s, "out", atts[s]))
            xn = modulated_layer_norm(x, shift2, scale2)
            return gated_residual(x, gate2, self._lin(s, "down", F.gelu(self._lin(s, "up", xn), approximate="tanh")))

        outs = self._on_two_streams(after_attention)
        return torch.cat([outs[s] for s in self.STREAMS], dim=1)


class BlockStack(nn.Module):
    """`n_blocks` double-stream blocks with one LoRA adapter set over every linear."""

    def __init__(self, n_blocks: int, cfg: BlockConfig, rank: int, alpha: float, device, seed: int = 5,
                 dtype: torch.dtype = torch.bfloat16, weight_copies="none", two_cuda_streams: bool = False):
        """`weight_copies`: "none" — every call dequantises into its workspace; "resident" (or True) —
        keep a bf16 copy of every frozen weight (2 bytes per element beside the packed 0.5), so that no
        call dequantises: the memory-for-time trade a 180 GB GPU allows; "block" — two arenas of one
        block's copies each, refilled one block ahead of the sweep on a side stream
        (`prefetch.BlockWeightPrefetcher`).  The one-token modulation sites never read a copy (their
        forward streams the packed bytes) and get none."""
        super().__init__()
        weight_copies = {True: "resident", False: "none", None: "none"}.get(weight_copies, weight_copies)
        if weight_copies not in ("none", "resident", "block"):
            raise ValueError(f"weight_copies must be none, resident or block, got {weight_copies!r}")
        self.weight_copies = weight_copies
        gen = torch.Generator(device=device).manual_seed(seed)
        self.cfg, self.dtype = cfg, dtype
        self.blocks = nn.ModuleList(DoubleStreamBlock(i, cfg, gen, device) for i in range(n_blocks))
        sites = [s for blk in self.blocks for s in blk.sites()]
        lcfg = LoraConfig(rank=rank, alpha=alpha, targets=[TargetSpec(r"^blocks\.")])
        torch.manual_seed(seed)  # identical adapters on every rank
        self.adapters = build_adapters(sites, lcfg, device)
        with torch.no_grad():  # non-zero B so that dA is exercised (crates/loractl-core/tests/block_ckpt.rs:69-71)
            g2 = torch.Generator(device=device).manual_seed(seed + 1)
            for d in self.adapters.deltas:
                d.lora_b.copy_(torch.randn(d.lora_b.shape, generator=g2, device=device) * 0.01)
        for blk in self.blocks:
            blk.adapters = self.adapters
            blk.two_cuda_streams = bool(two_cuda_streams)  # text and image chains of a block on two CUDA streams
            if weight_copies == "resident":
                for w in self._copy_weights(blk):
                    w.attach_bf16_copy()
        self.prefetcher = (BlockWeightPrefetcher([self._copy_weights(blk) for blk in self.blocks], device)
                           if weight_copies == "block" else None)
        self.flat = FlatAdapters(self.adapters, device)
        # slice of the flat buffers that holds block i's adapters (registration order = block order)
        per_block = 2 * len(DoubleStreamBlock.STREAMS) * len(DoubleStreamBlock.LINEARS)
        offs = self.flat.offsets + [self.flat.numel]
        self.block_slices = [(offs[i * per_block], offs[(i + 1) * per_block]) for i in range(n_blocks)]

    @staticmethod
    def _copy_weights(blk: DoubleStreamBlock):
        return [base.inner.weight for key, base in blk.bases.items() if not key.endswith("_mod")]

    def block_callables(self):
        """The blocks as `x -> x` callables for `checkpointed_step` / `forward`.  In "block" mode each
        one first makes its own weight copies current and starts the refill for the block the sweep
        visits next: i + 1 on the graph-free forward sweep, i - 1 while replaying for the backward."""
        if self.prefetcher is None:
            return list(self.blocks)
        pf = self.prefetcher

        def wrap(i, blk):
            def run(x):
                pf.acquire(i)
                pf.prefetch(i - 1 if torch.is_grad_enabled() else i + 1)
                return blk(x)
            return run

        return [wrap(i, blk) for i, blk in enumerate(self.blocks)]

    def lora_parameters(self):
        return [p for d in self.adapters.deltas for p in (d.lora_a, d.lora_b)]

    def set_cond(self, cond: torch.Tensor) -> None:
        for blk in self.blocks:
            blk.cond = cond

    def forward(self, state: torch.Tensor) -> torch.Tensor:
        for blk in self.block_callables():
            state = blk(state)
        return state


class GraphedSweep:
    """The block-checkpointed forward / head / reverse sweep of one step as CUDA graphs: one graph per
    block for the graph-free forward, one for the head (loss and its gradient), one per block for
    replay + backward — 2 L + 1 launches per step instead of some four hundred per block, so a small
    per-GPU batch is no longer bound by the host.  All graphs share one memory pool and are replayed
    in the order they were captured.  Static inputs: the trunk input, the conditioning vector, the
    regression target and the loss scale; each block's forward output is the next block's static
    input and stays alive as that block's checkpoint; adapter gradients go straight into the flat
    bucket (fixed addresses); the bf16 operand mirrors keep their buffers and are refreshed outside
    the graphs.  Captured for one batch shape; a different shape captures a new set.

    With `weight_copies="block"` the refill of the NEXT block's bf16 weight copies is a parallel branch
    inside the current block's graph (the dequantisation kernels of `attach_bf16_copy`, captured on a
    forked stream and joined at the end): forward graph i fills block i + 1, replay graph i fills block
    i - 1, each into the arena the sweep left two blocks ago.  Blocks 0 and 1 are filled once, eagerly:
    a sweep ends with exactly those two in place."""

    def __init__(self, stack: "BlockStack", state_shape, cond_shape, target_shape):
        dev = stack.flat.params.device
        self.stack = stack
        self.state = torch.zeros(state_shape, dtype=stack.dtype, device=dev)
        self.cond = torch.zeros(cond_shape, dtype=torch.bfloat16, device=dev)
        self.target = torch.zeros(target_shape, dtype=torch.float32, device=dev)
        self.loss_scale = torch.ones((), dtype=torch.float32, device=dev)
        self.stream = torch.cuda.Stream(device=dev)
        self.fwd, self.bwd, self.head = [], [], None
        self.loss = None

    def _head(self, s: torch.Tensor) -> torch.Tensor:
        li = self.stack.cfg.img_tokens
        return ((s[:, :li].float() - self.target) ** 2).mean()

    def capture(self) -> None:
        stack = self.stack
        blocks = list(stack.blocks)
        stack.set_cond(self.cond)
        stack.flat.refresh_mirrors()
        pf, n_blocks = stack.prefetcher, len(blocks)
        if pf is not None:  # the two blocks every sweep starts from, for real
            pf.release_all()
            pf.fill(0, torch.cuda.current_stream())
            if n_blocks > 1:
                pf.fill(1, torch.cuda.current_stream())
        # one eager pass on the capture stream: library plans, workspaces and side streams come into being here
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            x = self.state
            with torch.no_grad():
                for blk in blocks[:1] + blocks[-1:]:
                    x = blk(x)
            x2 = self.state.detach().requires_grad_(True)
            out = blocks[0](x2)
            (self._head(out) * self.loss_scale).backward()
        torch.cuda.current_stream().wait_stream(self.stream)
        torch.cuda.synchronize()
        stack.flat.zero_grad()
        pool = torch.cuda.graph_pool_handle()

        forked = [False]

        def refill(j: int) -> None:
            """Inside a capture: block j's copies rebuilt on the prefetch stream, beside the block's own work."""
            if pf is None or j < 0 or j >= n_blocks:
                return
            pf.stream.wait_stream(torch.cuda.current_stream())
            pf.fill(j, pf.stream)
            forked[0] = True

        def join() -> None:
            # only a stream that joined this capture may be waited for inside it
            if forked[0]:
                torch.cuda.current_stream().wait_stream(pf.stream)
                forked[0] = False

        inputs = [self.state]
        for i, blk in enumerate(blocks):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool, stream=self.stream, capture_error_mode="thread_local"):
                if 1 <= i <= n_blocks - 2:
                    refill(i + 1)
                with torch.no_grad():
                    out = blk(inputs[-1])
                join()
            self.fwd.append(g)
            inputs.append(out)
        self.head = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.head, pool=pool, stream=self.stream, capture_error_mode="thread_local"):
            x_final = inputs[-1].detach().requires_grad_(True)
            loss = self._head(x_final)
            (loss * self.loss_scale).backward()
            grad = x_final.grad
            self.loss = loss.detach()
        self.bwd = [None] * len(blocks)
        from . import quant as Q

        # what the graphs' kernels point at must outlive them: checkpoints, gradients, call workspaces
        self._keep = [inputs, grad, list(Q._workspaces.values())]
        for i in range(len(blocks) - 1, -1, -1):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool, stream=self.stream, capture_error_mode="thread_local"):
                if 1 <= i <= n_blocks - 2:
                    refill(i - 1)
                x2 = inputs[i].detach().requires_grad_(True)
                out = blocks[i](x2)
                out.backward(gradient=grad)
                grad = x2.grad
                join()
            self.bwd[i] = g
            self._keep.append(grad)
        if pf is not None:
            # the graphs carry the arena addresses; the handles themselves go back to per-call
            # dequantisation so that eager calls outside the graphs stay correct
            pf.release_all()
        stack.flat.zero_grad()  # the captures themselves ran nothing, but keep the bucket's state obvious

    def run(self, state: torch.Tensor, cond: torch.Tensor, target: torch.Tensor, loss_scale: float, after_block) -> torch.Tensor:
        self.state.copy_(state)
        self.cond.copy_(cond)
        self.target.copy_(target)
        self.loss_scale.fill_(loss_scale)
        for g in self.fwd:
            g.replay()
        self.head.replay()
        for i in range(len(self.bwd) - 1, -1, -1):
            self.bwd[i].replay()
            after_block(i)
        return self.loss


class GraphedLossStep:
    """`loss = fn(); loss.backward()` captured once as ONE CUDA graph and replayed: for a model that is
    stepped without block checkpointing (the text model: 12 small layers, ~2,500 launches per step).
    `fn` must read its inputs from fixed tensors (copy new data into them before `replay`), the
    adapter gradients must accumulate into fixed memory (a `FlatAdapters` bucket), and the bf16 factor
    mirrors must be refreshed outside the graph after every optimizer step."""

    def __init__(self, fn, device, warm: int = 1):
        self.stream = torch.cuda.Stream(device=device)
        cur = torch.cuda.current_stream(device)
        self.stream.wait_stream(cur)
        with torch.cuda.stream(self.stream):  # plans, workspaces and side streams come into being here
            for _ in range(max(warm, 1)):
                fn().backward()
        cur.wait_stream(self.stream)
        torch.cuda.synchronize(device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=self.stream, capture_error_mode="thread_local"):
            loss = fn()
            loss.backward()
            self.loss = loss.detach()
        from . import quant as Q

        self._keep = list(Q._workspaces.values())

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.loss


class Trainer:
    """One rank of the data-parallel LoRA trainer over a `BlockStack`."""

    def __init__(self, stack: BlockStack, lr: float = 1e-4, weight_decay: float = 1e-4, group=None,
                 grad_checkpointing: bool = True, graphs: bool = False, reduce_every: int = 1):
        """`graphs`: run the checkpointed sweep as CUDA graphs (`GraphedSweep`), captured at the first
        step of each batch shape.  `reduce_every`: blocks per gradient all-reduce of the reverse sweep
        (1 = one slice per block, started as soon as that block's backward is enqueued; the number of
        blocks = one all-reduce of the whole bucket after the sweep)."""
        self.stack, self.lr, self.group = stack, lr, group
        self.optim = AdamW(stack.flat, weight_decay=weight_decay)
        self.scaler = DynamicLossScale(initial=1.0)  # bf16/f32 gradients do not need the f16 head-room
        self.grad_checkpointing = grad_checkpointing
        if graphs and not grad_checkpointing:
            raise ValueError("graphs=True captures the block-checkpointed sweep: it needs grad_checkpointing")
        self.graphs = graphs
        self.reduce_every = max(int(reduce_every), 1)
        self._sweeps = {}
        self.steps_done = 0

    def step(self, x0: torch.Tensor, txt: torch.Tensor, cond: torch.Tensor, t: torch.Tensor,
             noise: torch.Tensor) -> float:
        """x0 [b, L_img, h] clean latents, txt [b, L_txt, h], cond [b, h], t [b] in (0, 1), noise like x0.
        Flow matching (crates/loractl-core/src/flow.rs:50-66): x_t = (1 - t) x0 + t eps, target
        v = eps - x0, loss = mean((pred - v)^2) over the image tokens."""
        stack, flat = self.stack, self.stack.flat
        tt = t.view(-1, 1, 1).to(x0.dtype)
        x_t = (1 - tt) * x0 + tt * noise
        target = (noise - x0).float()
        li = stack.cfg.img_tokens
        stack.set_cond(cond)
        state = torch.cat([x_t, txt], dim=1).to(stack.dtype)
        head = lambda s: ((s[:, :li].float() - target) ** 2).mean()
        flat.zero_grad()
        params = stack.lora_parameters()
        reducer = dp.BucketReducer(flat.grads, self.group)
        # a block's gradients are final once its replayed backward is enqueued: their all-reduce
        # starts there and overlaps the replay of the blocks below it
        n_blocks = len(stack.blocks)

        def after_block(i: int) -> None:
            if reducer.world > 1:
                flat.gather_autograd_grads(stack.block_slices[i])
                due = dp.sweep_reduce_range(n_blocks, self.reduce_every, i)
                if due is not None:
                    reducer.reduce_slice(stack.block_slices[due[0]][0], stack.block_slices[due[1]][1])

        torch.cuda.nvtx.range_push("lq.sweep")  # forward, head, reverse sweep (+ per-block all-reduce starts)
        if self.graphs:
            key = (tuple(state.shape), tuple(cond.shape))
            sweep = self._sweeps.get(key)
            if sweep is None:
                sweep = GraphedSweep(stack, state.shape, cond.shape, target.shape)
                sweep.capture()
                self._sweeps[key] = sweep
            stack.set_cond(sweep.cond)
            loss_dev = sweep.run(state, cond, target, self.scaler.loss_scale, after_block)
            flat.gather_autograd_grads()
        elif self.grad_checkpointing:
            loss, _ = checkpointed_step(stack.block_callables(), state, head, params, self.scaler.loss_scale,
                                        keep_existing_grads=True, after_block=after_block)
            flat.gather_autograd_grads()
        else:
            loss_t = head(stack(state))
            (loss_t * self.scaler.loss_scale).backward()
            loss = float(loss_t.detach())
            flat.gather_autograd_grads()
            reducer.reduce_slice(0, flat.numel)
        torch.cuda.nvtx.range_pop()
        # non-finite values survive the sum, so the flag is taken on the reduced gradients
        torch.cuda.nvtx.range_push("lq.reduce_finish")
        scale = reducer.finish()
        torch.cuda.nvtx.range_pop()
        torch.cuda.nvtx.range_push("lq.optimizer")
        nonfinite_flag(flat.grads, flat.flag)
        dp.reduce_flag(flat.flag, self.group)
        # the optimizer reads the flag on the device and skips itself; the host reads it only to
        # advance the loss-scale state (where the reference reads its |g| sum back)
        self.optim.step(self.lr, grad_scale=scale / self.scaler.loss_scale, skip_flag=flat.flag)
        flat.refresh_mirrors()  # the factors changed: all bf16 operand mirrors in one batched launch
        torch.cuda.nvtx.range_pop()
        if self.graphs:
            loss = float(loss_dev)
        finite, _ = dp.consensus_step(self.scaler, flat.flag)
        if not finite:
            self.optim.steps -= 1  # a skipped update does not advance the bias-correction clock
        self.steps_done += 1
        return loss

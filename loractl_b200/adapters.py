"""Name-keyed adapter set — the mirror of crates/loractl-core/src/adapters.rs."""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
from torch import nn

from .lora import LoraDelta


@dataclass(frozen=True)
class LoraSite:
    """crates/loractl-core/src/adapters.rs:94-103."""

    path: str
    d_in: int
    d_out: int


@dataclass
class TargetSpec:
    """crates/loractl-core/src/config.rs `TargetSpec`: a regex plus optional per-target overrides."""

    pattern: str
    rank: Optional[int] = None
    alpha: Optional[float] = None


@dataclass
class LoraConfig:
    rank: int = 8
    alpha: float = 8.0
    dropout: float = 0.0
    targets: Sequence[TargetSpec] = ()


class LoraAdapters(nn.Module):
    """crates/loractl-core/src/adapters.rs:46-85: `deltas[i]` adapts the layer at `targets[i]`."""

    def __init__(self, deltas: Sequence[LoraDelta] = (), targets: Sequence[str] = ()):
        super().__init__()
        if len(deltas) != len(targets):
            raise ValueError("deltas and targets must stay in lockstep")
        self.deltas = nn.ModuleList(deltas)
        self.targets: List[str] = list(targets)

    def get(self, path: str) -> Optional[LoraDelta]:
        """Linear scan over `targets` (adapters.rs:62-67)."""
        for i, t in enumerate(self.targets):
            if t == path:
                return self.deltas[i]
        return None

    def apply(self, path: str, x: torch.Tensor, base_out: torch.Tensor) -> torch.Tensor:
        """adapters.rs:75-85: `base_out + delta.forward(x)` when a delta targets `path`.
        (Sites with a quantized base do not come through here: `linear.site` fuses the delta
        into the base kernel.)"""
        d = self.get(path)
        return base_out if d is None else base_out + d(x)


def build_adapters(sites: Sequence[LoraSite], cfg: LoraConfig, device=None) -> LoraAdapters:
    """crates/loractl-core/src/adapters.rs:116-145: first matching target pattern wins; per-target
    rank/alpha override the globals; registration order follows `sites`.  An invalid regex
    raises immediately."""
    compiled = []
    for spec in cfg.targets:
        try:
            compiled.append((re.compile(spec.pattern), spec))
        except re.error as e:
            raise ValueError(f"invalid LoRA target pattern {spec.pattern!r}: {e}") from e
    deltas, targets = [], []
    for site in sites:
        for rx, spec in compiled:
            if rx.search(site.path):
                rank = spec.rank if spec.rank is not None else cfg.rank
                alpha = spec.alpha if spec.alpha is not None else cfg.alpha
                deltas.append(LoraDelta(site.d_in, site.d_out, rank, alpha, cfg.dropout, device))
                targets.append(site.path)
                break
    return LoraAdapters(deltas, targets)

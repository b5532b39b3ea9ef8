"""Boundary vocabulary — the slice of crates/loractl-core/src/config.rs this backend touches:
`compute.backend` gains one spelling, `b200`, and the quant guard matrix of
crates/loractl-core/src/diffusion_trainer.rs:377-401 gains one row."""
from __future__ import annotations

import enum
from dataclasses import dataclass

from .quant import Quant


class BackendKind(enum.Enum):
    """config.rs:515-529 plus `B200`."""

    NDARRAY = "ndarray"
    WGPU = "wgpu"
    CANDLE = "candle"
    CUDA = "cuda"
    TCH = "tch"
    B200 = "b200"

    @staticmethod
    def parse(s: str) -> "BackendKind":
        k = s.lower()
        if k == "libtorch":
            k = "tch"
        for b in BackendKind:
            if b.value == k:
                return b
        raise ValueError(f"unknown backend {s!r} (ndarray|wgpu|candle|cuda|tch|b200)")


class Precision(enum.Enum):
    """config.rs:576-590 (`f32`, `f16`, `bf16`)."""

    F32 = "f32"
    F16 = "f16"
    BF16 = "bf16"

    @staticmethod
    def parse(s: str) -> "Precision":
        k = s.lower()
        if k in ("f32", "fp32", "full"):
            return Precision.F32
        if k in ("f16", "fp16", "half"):
            return Precision.F16
        if k in ("bf16", "bfloat16"):
            return Precision.BF16
        raise ValueError(f"unknown precision {s!r} (f32|f16|bf16)")


DEFAULT_DEQUANT_CHUNK_MIB = 512  # config.rs:688


@dataclass
class ComputeConfig:
    backend: BackendKind = BackendKind.NDARRAY
    device: int = 0
    precision: Precision = Precision.F32
    grad_checkpointing: bool = False
    quant: Quant = Quant.NONE
    dequant_chunk_mib: int = DEFAULT_DEQUANT_CHUNK_MIB


def validate_b200(compute: ComputeConfig, lora_dropout: float = 0.0) -> None:
    """The b200 row of the guard matrix.  Every rejected combination raises with a named
    reason; nothing falls back to another backend or to the CPU."""
    if compute.backend is not BackendKind.B200:
        raise ValueError(f"this library implements compute.backend = b200, got {compute.backend.value}")
    if compute.precision is Precision.F16:
        raise ValueError("compute.precision = f16 is not supported on b200; use f32 (reference numerics) or bf16 "
                         "(tcgen05 tensor cores)")
    if compute.grad_checkpointing and lora_dropout > 0.0:
        # diffusion_trainer.rs:342-348: a replay would redraw dropout masks
        raise ValueError("compute.grad_checkpointing is incompatible with lora.dropout > 0")
    if compute.quant is not Quant.NONE and lora_dropout > 0.0:
        raise ValueError("lora.dropout > 0 is not supported on quantized sites of the b200 backend")

"""loractl_b200 — the B200 (sm_100a) backend of loractl's quantized frozen-base LoRA linear.

The package holds only what that path needs: the CUDA library (`csrc/`, built into
`lib/libloractl_b200.so`) and a host-side mirror of the reference's interface for it
(quant.rs, lora.rs, adapters.rs, the QuantLinear / BaseLinear / site part of mmdit.rs,
fp8.rs, block_ckpt.rs)."""
from .quant import (QUANT_BLOCK, Quant, QuantWeight, check_device_status, dequant_chunk_rows, quant_matmul_t,
                    quant_value, quantize_linear_weight, quantize_linear_weight_chunked)
from .lora import LoraDelta, LoraLinear, init_factors
from .adapters import LoraAdapters, LoraConfig, LoraSite, TargetSpec, build_adapters
from .linear import BaseLinear, QuantLinear, site
from .fp8 import e4m3fn_lut, fp8_quantize, weight_from_fp8
from .config import BackendKind, ComputeConfig, Precision, validate_b200
from .optim import AdamW, DynamicLossScale, FlatAdapters, nonfinite_flag
from .block_ckpt import checkpointed_step
from . import dp, export, loader
from .export import export_adapters, import_adapters
from .loader import load_quant_module

__all__ = [
    "QUANT_BLOCK", "Quant", "QuantWeight", "check_device_status", "dequant_chunk_rows", "quant_matmul_t",
    "quant_value", "quantize_linear_weight", "quantize_linear_weight_chunked",
    "LoraDelta", "LoraLinear", "init_factors", "LoraAdapters", "LoraConfig", "LoraSite", "TargetSpec",
    "build_adapters", "BaseLinear", "QuantLinear", "site", "e4m3fn_lut", "fp8_quantize", "weight_from_fp8",
    "BackendKind", "ComputeConfig", "Precision", "validate_b200",
    "AdamW", "DynamicLossScale", "FlatAdapters", "nonfinite_flag", "checkpointed_step", "dp",
    "export", "loader", "export_adapters", "import_adapters", "load_quant_module",
]

"""ctypes binding of libloractl_b200.so (the C ABI declared in include/loractl_b200.h).

There is no CPU fallback: if the shared library is missing the import fails
with instructions to build it, and every failing call raises `LqError` with
the library's own message (crates/loractl-core/src/config.rs:503-512: fail
loudly, never fall back).
"""
from __future__ import annotations

import ctypes as C
import pathlib

LIB_PATH = pathlib.Path(__file__).resolve().parent / "lib" / "libloractl_b200.so"

LQ_OK, LQ_ERR_INVALID, LQ_ERR_CUDA, LQ_ERR_UNSUPPORTED, LQ_ERR_TIMEOUT, LQ_ERR_WORKSPACE = range(6)
LQ_F32, LQ_BF16, LQ_BF16_W8A8 = 0, 1, 2
LQ_INT4, LQ_INT8, LQ_FP8_E4M3 = 4, 8, 108
LQ_SCALE_SCALAR, LQ_SCALE_PER_CHANNEL = 0, 1


class LqError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"loractl_b200 error {status}: {message}")
        self.status = status
        self.message = message


class GroupSite(C.Structure):
    """`lq_group_site` of include/loractl_b200.h."""
    _fields_ = [("w", C.c_void_p), ("A", C.c_void_p), ("B", C.c_void_p), ("rank", C.c_int32), ("scaling", C.c_float),
                ("Y", C.c_void_p), ("H_out", C.c_void_p)]


class MirrorJob(C.Structure):
    """`lq_mirror_job` of include/loractl_b200.h."""
    _fields_ = [("A", C.c_void_p), ("B", C.c_void_p), ("d_in", C.c_int64), ("d_out", C.c_int64), ("rank", C.c_int32),
                ("mirror", C.c_void_p)]


class WeightInfo(C.Structure):
    _fields_ = [
        ("d_out", C.c_int64), ("d_in", C.c_int64), ("scheme", C.c_int32), ("group", C.c_int32),
        ("scale_kind", C.c_int32), ("has_bias", C.c_int32), ("device", C.c_int32), ("reserved", C.c_int32),
        ("packed_bytes", C.c_uint64), ("scale_bytes", C.c_uint64),
    ]


_P, _I, _I64, _F, _SZ = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); exactly the symbols include/loractl_b200.h declares
SIGNATURES = {
    "lq_last_error": (C.c_char_p, []),
    "lq_abi_version": (_I, []),
    "lq_dequant_chunk_rows": (_I, [C.c_uint64, C.c_uint64, C.c_uint64, C.POINTER(C.c_uint64), _SZ, C.POINTER(_SZ)]),
    "lq_quantize": (_I, [_P, _I, _I64, _I64, _I, _I, _P, C.POINTER(_P)]),
    "lq_weight_from_codes": (_I, [_P, _P, _I64, _I64, _I, _I, _P, C.POINTER(_P)]),
    "lq_weight_from_fp8": (_I, [_P, _P, _I, _I64, _I64, _P, C.POINTER(_P)]),
    "lq_quantize_from_fp8": (_I, [_P, _P, _I, _I64, _I64, _I, _I, _P, C.POINTER(_P)]),
    "lq_fp8_quantize": (_I, [_P, _I64, _I64, _I, _P, C.POINTER(_P)]),
    "lq_weight_set_bias": (_I, [_P, _P, _P]),
    "lq_weight_info_get": (_I, [_P, C.POINTER(WeightInfo)]),
    "lq_weight_destroy": (_I, [_P]),
    "lq_unpack": (_I, [_P, _P, _P, _P]),
    "lq_dequantize": (_I, [_P, _P, _I, _P]),
    "lq_linear_workspace_bytes": (_SZ, [_P, _I64, _I, _I]),
    "lq_linear_fwd": (_I, [_P, _P, _I64, _I, _P, _P, _I, _F, _P, _P, _P, _SZ, _P, _P]),
    "lq_linear_bwd": (_I, [_P, _P, _P, _P, _I64, _I, _P, _P, _I, _F, _P, _P, _P, _I, _P, _SZ, _P, _P]),
    "lq_weight_bf16_copy_bytes": (_SZ, [_P]),
    "lq_weight_attach_bf16_copy": (_I, [_P, _P, _P]),
    "lq_lora_mirror_bytes": (_SZ, [_I64, _I64, _I]),
    "lq_lora_mirror_update": (_I, [_P, _P, _I64, _I64, _I, _P, _P]),
    "lq_lora_mirror_update_batch": (_I, [_P, _I, _P]),
    "lq_linear_grouped_workspace_bytes": (_SZ, [C.POINTER(GroupSite), _I, _I64, _I]),
    "lq_linear_fwd_grouped": (_I, [C.POINTER(GroupSite), _I, _P, _I64, _I, _P, _SZ, _P]),
    "lq_weight_prepare_fp8_backward": (_I, [_P, _P]),
    "lq_grad_nonfinite_flag": (_I, [_P, _I64, _P, _P]),
    "lq_adamw_step": (_I, [_P, _P, _P, _P, _I64, _F, _F, _F, _F, _F, _I64, _F, _P, _P]),
    "lq_block_ops_workspace_bytes": (C.c_size_t, [_I64, _I64, _I64]),
    "lq_ln_modulate_fwd": (_I, [_P, _P, _P, _I, _I64, _I64, _I64, C.c_float, _P, _P, _P, _P]),
    "lq_ln_modulate_bwd": (_I, [_P, _P, _P, _P, _P, _I, _I64, _I64, _I64, _P, _P, _P, _P, C.c_size_t, _P]),
    "lq_gate_residual_fwd": (_I, [_P, _P, _P, _I, _I64, _I64, _I64, _P, _P]),
    "lq_zrmsnorm_fwd": (_I, [_P, _P, _I, _I64, _I64, _F, _P, _P, _P]),
    "lq_zrmsnorm_bwd": (_I, [_P, _P, _P, _P, _I, _I64, _I64, _P, _P]),
    "lq_swiglu_fwd": (_I, [_P, _P, _I, _I64, _P, _P]),
    "lq_swiglu_bwd": (_I, [_P, _P, _P, _I, _I64, _P, _P, _P]),
    "lq_sigmoid_gate_fwd": (_I, [_P, _P, _I, _I64, _P, _P]),
    "lq_sigmoid_gate_bwd": (_I, [_P, _P, _P, _I, _I64, _P, _P, _P]),
    "lq_gate_residual_bwd": (_I, [_P, _P, _P, _I, _I64, _I64, _I64, _P, _P, _P, C.c_size_t, _P]),
    "lq_check_device_status": (_I, [_P]),
    "lq_selftest_bounded_wait": (_I, [C.c_uint, _P]),
    "lq_kernel_launch_count": (C.c_uint64, []),
    "lq_profile_enable": (_I, [_I]),
    "lq_profile_kinds": (_I, []),
    "lq_profile_kind_name": (C.c_char_p, [_I]),
    "lq_profile_collect": (_I, [C.POINTER(C.c_double), C.POINTER(C.c_uint64), _I]),
    "lq_gemm_bf16_splitk_static": (_I, [_P, _P, _I, _I64, _I64, _P, _I64, _I64, _I64, _I64, _I, _P]),
    "lq_option_set": (_I, [C.c_char_p, _I]),
    "lq_gemm_bf16": (_I, [_P, _I, _I64, _P, _I, _I64, _P, _I, _I64, _I64, _I64, _I64, _I, _I, _P, _P, _P]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m loractl_b200._build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this backend."
            )
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != LQ_OK:
        raise LqError(status, lib().lq_last_error().decode("utf-8", "replace"))

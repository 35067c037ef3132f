"""ctypes binding of libaklr_b200.so (the C ABI declared in include/aklr_b200.h).

The library is built in-tree by ``aklr_b200.csrc.build``; loading fails loudly when it is
missing -- there is no CPU or eager fallback behind these calls.
"""

from __future__ import annotations

import ctypes
import pathlib
from ctypes import POINTER, c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p

LIB_PATH = pathlib.Path(__file__).resolve().parent / "libaklr_b200.so"

SCORING = {"softmax": 0, "sigmoid": 1}
DTYPE_BF16, DTYPE_F32 = 0, 1
# aklr_moe_config.variant bits (AKLR_VARIANT_* of the header)
VARIANT_WEIGHT_MAJOR, VARIANT_CTA_PAIRS, VARIANT_SEPARATE_PROLOGUE, VARIANT_FULL_ACTIVATION_BOXES = 1, 2, 4, 8
VARIANT_BF16_ACTIVATIONS, VARIANT_MXFP4_ACTIVATIONS = 16, 32  # numerics modes of the MXFP4 entry points
VARIANT_DEEP_PIPELINE = 64
VARIANT_TILED_WEIGHTS = 128  # w1 / w2 in the tile-contiguous layout


class AklrError(RuntimeError):
    """A call into libaklr_b200.so returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libaklr_b200: {message} (status {code})")
        self.code = code


class MoeConfig(ctypes.Structure):
    _fields_ = [
        ("n_tokens", c_int32),
        ("hidden", c_int32),
        ("inter", c_int32),
        ("n_routed", c_int32),
        ("n_shared", c_int32),
        ("topk", c_int32),
        ("scoring", c_int32),
        ("num_expert_group", c_int32),
        ("topk_group", c_int32),
        ("renormalize", c_int32),
        ("routed_scaling_factor", c_float),
        ("logits_dtype", c_int32),
        ("bias_dtype", c_int32),
        ("block_m", c_int32),
        ("n_experts_global", c_int32),
        ("variant", c_int32),
    ]


class MxOptions(ctypes.Structure):
    """``aklr_mx_options`` of the public header."""

    _fields_ = [
        ("activation", c_int32),
        ("weight_in_stage1", c_int32),
        ("swiglu_limit", c_float),
        ("beta", c_float),
        ("linear_beta", c_float),
        ("num_local_tokens", c_void_p),
    ]


class WorkspaceLayout(ctypes.Structure):
    _fields_ = [(name, c_int64) for name in (
        "total_bytes", "status", "topk_ids", "topk_weights", "sorted_ids", "block_expert", "counts",
        "num_blocks", "chunk_hist", "xq", "xs", "hq", "hs", "rows")] + [
        ("block_m", c_int32), ("max_blocks", c_int32), ("capacity", c_int32), ("n_experts", c_int32)]


# name -> (restype, argtypes): every symbol include/aklr_b200.h declares
SIGNATURES = {
    "aklr_abi_version": (c_int32, []),
    "aklr_status_string": (c_char_p, [c_int32]),
    "aklr_last_error": (c_char_p, []),
    "aklr_moe_fp8_workspace": (c_int32, [POINTER(MoeConfig), POINTER(WorkspaceLayout)]),
    "aklr_moe_fp8_forward": (c_int32, [POINTER(MoeConfig)] + [c_void_p] * 9 + [c_void_p, c_size_t, c_void_p]),
    "aklr_moe_fp8_experts": (c_int32, [POINTER(MoeConfig)] + [c_void_p] * 9 + [c_void_p, c_size_t, c_void_p]),
    "aklr_moe_mxfp4_experts": (c_int32, [POINTER(MoeConfig)] + [c_void_p] * 8 + [c_float, c_void_p, c_void_p, c_size_t, c_void_p]),
    "aklr_moe_mxfp4_experts_ex": (c_int32, [POINTER(MoeConfig)] + [c_void_p] * 8 + [POINTER(MxOptions), c_void_p, c_void_p, c_size_t, c_void_p]),
    "aklr_moe_mxfp4_forward": (c_int32, [POINTER(MoeConfig)] + [c_void_p] * 8 + [c_float, c_void_p, c_void_p, c_size_t, c_void_p]),
    "aklr_ep_gather_quant_mxfp8": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p]),
    "aklr_moe_mxfp4_experts_prequant": (c_int32, [POINTER(MoeConfig)] + [c_void_p] * 8 + [c_float, c_void_p, c_void_p, c_size_t, c_void_p]),
    "aklr_ep_gather_rows": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p]),
    "aklr_ep_gather_quant": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p]),
    "aklr_ep_dispatch_meta": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p]),
    "aklr_moe_fp8_experts_prequant": (c_int32, [POINTER(MoeConfig)] + [c_void_p] * 9 + [c_void_p, c_size_t, c_void_p]),
    "aklr_ep_combine": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p]),
    "aklr_ep_counts_to_host": (c_int32, [c_void_p, c_void_p, c_int32, c_void_p, c_void_p]),
    "aklr_ep_row_bytes": (c_int32, [c_int32, c_int32, c_int32]),
    "aklr_ep_plan": (c_int32, [c_void_p, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p]),
    "aklr_ep_pack": (c_int32, [c_void_p] * 5 + [c_int32] * 6 + [c_void_p, c_void_p, c_void_p, c_void_p]),
    "aklr_ep_unpack_meta": (c_int32, [c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p]),
    "aklr_moe_fp8_experts_rows": (c_int32, [POINTER(MoeConfig), c_void_p, c_int32, c_void_p, c_int32] + [c_void_p] * 7 + [c_void_p, c_size_t, c_void_p]),
    "aklr_moe_mxfp4_experts_rows": (c_int32, [POINTER(MoeConfig), c_void_p, c_int32, c_void_p, c_int32] + [c_void_p] * 6 + [c_float, c_void_p, c_void_p, c_size_t, c_void_p]),
    "aklr_moe_route": (c_int32, [POINTER(MoeConfig)] + [c_void_p] * 5 + [c_void_p]),
    "aklr_moe_align": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32] + [c_void_p] * 5 + [c_void_p]),
    "aklr_moe_align_max_blocks": (c_int64, [c_int64, c_int64, c_int64]),
    "aklr_moe_align_noalloc": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32] + [c_void_p] * 4 + [c_void_p]),
    "aklr_moe_align_noalloc_max_scratch_ints": (c_int32, []),
    "aklr_moe_align_noalloc_last_error": (c_char_p, []),
    "aklr_silu_mul_bf16": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_void_p]),
    "aklr_moe_add_gated_rows": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_void_p]),
    "aklr_selftest_exact_divide": (c_int32, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "aklr_tile_weights_fp8": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, c_int32, c_void_p]),
    "aklr_moe_shared_gate": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "aklr_router_gemm_f32": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p]),
    "aklr_router_gemm_bf16": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p]),
    "aklr_per_group_quant_fp8": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_void_p]),
    "aklr_per_group_quant_mxfp8": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_void_p]),
    "aklr_moe_act_quant_fp8": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_void_p]),
    "aklr_moe_read_status": (c_int32, [c_void_p, POINTER(c_int32), c_void_p]),
    "aklr_kernel_launch_count": (c_int64, []),
    "aklr_device_status": (c_int32, [POINTER(c_int32), c_int32]),
    "aklr_selftest_wait_expiry": (c_int32, [c_int64, c_void_p, c_void_p]),
    "aklr_profile_begin": (c_int32, [c_int32]),
    "aklr_profile_read": (c_int32, [c_int32, POINTER(c_float)]),
}

_lib = None


def load() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m aklr_b200.csrc.build` "
                "(there is no fallback path for the fused-MoE kernels)"
            )
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = lib
    return _lib


def check(code: int) -> None:
    if code != 0:
        raise AklrError(code, load().aklr_last_error().decode() or load().aklr_status_string(code).decode())

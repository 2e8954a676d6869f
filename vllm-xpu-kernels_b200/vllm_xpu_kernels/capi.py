"""ctypes view of the C ABI declared in include/b200moe.h.

For callers (and tests) that hold raw device pointers instead of torch
tensors.  Every function returns the library's integer status.
"""
import ctypes
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t,
                    c_void_p)

from ._loader import CAPI_PATH

OK, INVALID_ARG, UNSUPPORTED, WORKSPACE_TOO_SMALL, CUDA_ERROR, TIMEOUT = 0, -1, -2, -3, -4, -5
EP_BARRIER_CHANNELS = 4   # B200MOE_EP_BARRIER_CHANNELS of include/b200moe.h
F32, F16, BF16, E4M3, I32, I64, U32, U8, E2M1X2 = range(9)
RECIPE_BF16, RECIPE_FP8_BLOCK, RECIPE_MXFP4 = 0, 1, 2
B_LAYOUT_KN, B_LAYOUT_NK = 0, 1
EPI_STORE, EPI_SILU_MUL, EPI_SWIGLU_OAI = 0, 1, 2


class GemmArgs(Structure):
    _fields_ = [
        ("recipe", c_int), ("epilogue", c_int), ("a_dtype", c_int), ("d_dtype", c_int),
        ("A", c_void_p), ("a_scale", c_void_p), ("B", c_void_p), ("b_layout", c_int),
        ("b_scale", c_void_p), ("bias", c_void_p), ("bias_dtype", c_int), ("D", c_void_p),
        ("d_scale", c_void_p), ("rows_per_expert", c_void_p), ("R", c_int64), ("N", c_int),
        ("K", c_int), ("E", c_int), ("alpha", c_float), ("limit", c_float), ("d_row_ptr", c_void_p),
        ("a_scale_layout", c_int), ("gated_act", c_int), ("act_param0", c_float),
        ("act_param1", c_float), ("clamp_limit", c_float), ("scales_pow2", c_int),
    ]


class MxGemmArgs(Structure):
    _fields_ = [
        ("epilogue", c_int), ("d_dtype", c_int), ("A", c_void_p), ("a_sf", c_void_p),
        ("a_sf_pitch", c_int64), ("B", c_void_p), ("b_sf", c_void_p), ("bias", c_void_p),
        ("bias_dtype", c_int), ("D", c_void_p), ("d_sf", c_void_p), ("d_sf_pitch", c_int64),
        ("rows_per_expert", c_void_p), ("R", c_int64), ("N", c_int), ("K", c_int), ("E", c_int),
        ("alpha", c_float), ("limit", c_float),
    ]


# name -> (restype, argtypes); must list every symbol include/b200moe.h declares.
SIGNATURES = {
    "b200moe_version": (c_char_p, []),
    "b200moe_status_string": (c_char_p, [c_int]),
    "b200moe_last_error": (c_char_p, []),
    "b200moe_launch_count": (ctypes.c_longlong, []),
    "b200moe_topk_softmax": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "b200moe_topk_sigmoid": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                     c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                     c_void_p]),
    "b200moe_grouped_topk": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p]),
    "b200moe_moe_align_block_size_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "b200moe_moe_align_block_size": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_void_p,
                                             c_void_p, c_int64, c_void_p, c_int64, c_void_p,
                                             c_void_p, c_size_t, c_void_p]),
    "b200moe_moe_align_block_size_static": (c_int, [c_void_p, c_int, c_int64, c_int, c_int,
                                                    c_void_p, c_void_p, c_int64, c_void_p,
                                                    c_int64, c_void_p, c_void_p]),
    "b200moe_init_expert_map": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200moe_remap_hidden_states_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "b200moe_remap_hidden_states": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                            c_int64, c_void_p, c_int, c_void_p, c_int, c_int,
                                            c_int, c_int, c_void_p, c_void_p, c_void_p, c_size_t,
                                            c_void_p]),
    "b200moe_moe_gather": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                   c_int, c_void_p]),
    "b200moe_moe_gather_add": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                       c_int, c_int, c_void_p]),
    "b200moe_moe_sum": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                c_void_p, c_void_p]),
    "b200moe_moe_lora_align_block_size": (c_int, [c_void_p, c_int, c_int64, c_int, c_void_p, c_int,
                                                  c_int, c_int, c_int64, c_int64, c_void_p,
                                                  c_void_p, c_void_p, c_void_p, c_void_p,
                                                  c_void_p, c_void_p]),
    "b200moe_act_and_mul": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_float,
                                    c_float, c_float, c_void_p]),
    "b200moe_expand_weights": (c_int, [c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                                       c_int, c_int, c_int, c_int, c_void_p]),
    "b200moe_silu_and_mul": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_void_p]),
    "b200moe_swigluoai_and_mul": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_float,
                                          c_float, c_void_p]),
    "b200moe_per_token_group_fp8_quant": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64,
                                                  c_int, c_int, c_float, c_float, c_float, c_int,
                                                  c_int64, c_int64, c_void_p]),
    "b200moe_per_token_group_quant_mxfp4": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64,
                                                    c_int, c_int, c_float, c_int64, c_int64,
                                                    c_void_p]),
    "b200moe_silu_mul_block_quant": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int,
                                             c_int, c_void_p, c_int, c_int64, c_int64, c_void_p]),
    "b200moe_silu_mul_mxfp4_quant": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int,
                                             c_int, c_float, c_void_p]),
    "b200moe_grouped_gemm_workspace_bytes": (c_size_t, [POINTER(GemmArgs)]),
    "b200moe_grouped_gemm": (c_int, [POINTER(GemmArgs), c_void_p, c_size_t, c_void_p]),
    "b200moe_dequant_weights": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                        c_void_p]),
    "b200moe_mx_weight_scales_bytes": (c_size_t, [c_int, c_int, c_int]),
    "b200moe_mx_prepare_weight_scales": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200moe_quant_mxfp8": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_int64,
                                    c_void_p]),
    "b200moe_grouped_gemm_mx": (c_int, [POINTER(MxGemmArgs), c_void_p]),
    "b200moe_grouped_gemm_check": (c_int, [POINTER(GemmArgs), c_void_p]),
    "b200moe_device_status": (c_int, [c_void_p, POINTER(c_int)]),
    "b200moe_selftest_wait_timeout": (c_int, [ctypes.c_longlong, c_void_p]),
    "b200moe_topk_softplus_sqrt": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                           c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_int, c_void_p, c_void_p]),
    "b200moe_batched_moe_align_block_size": (c_int, [c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                                     c_void_p, c_void_p]),
    "b200moe_reorder_mxfp_scales": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p,
                                            c_void_p]),
    "b200moe_ep_barrier": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_int64, c_void_p]),
    "b200moe_ep_barrier_emulated": (c_int, [c_void_p, c_void_p, c_int, c_int, ctypes.c_uint32, c_int64,
                                            c_void_p]),
    "b200moe_ep_rank_hits": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200moe_ep_pack_routing": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
                                        c_void_p]),
    "b200moe_ep_unpack_routing": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                                          c_void_p, c_void_p, c_void_p]),
    "b200moe_moe_gather_bounded": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                           c_int, c_int, c_int, c_void_p]),
    "b200moe_ep_put_counts": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "b200moe_ep_offsets": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p]),
    "b200moe_ep_push": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int,
                                c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                c_void_p]),
    "b200moe_ep_dispatch": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int, c_void_p,
                                    c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                    c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "b200moe_ep_source_table": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_int64,
                                        c_int64, c_int64, c_void_p, c_void_p]),
    "b200moe_ep_gather": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                  c_void_p]),
    "b200moe_ep_return_table": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64,
                                        c_void_p, c_void_p]),
}

_lib = None


def lib():
    """The loaded library with argument types set."""
    global _lib
    if _lib is None:
        handle = ctypes.CDLL(CAPI_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def status_string(code: int) -> str:
    return lib().b200moe_status_string(code).decode()

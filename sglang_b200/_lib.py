"""ctypes binding of libb200_block_fp8.so (the C ABI declared in include/b200_block_fp8.h).

There is no CPU or PyTorch fallback: if the library is missing or a call fails, this raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libb200_block_fp8.so")

DT_F32, DT_F16, DT_BF16 = 0, 1, 2

_lib = None


class B200Error(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, fn: str, code: int, detail: str):
        super().__init__(f"{fn}: {detail} (code {code})")
        self.code = code


_SIGNATURES = {
    "b200_strerror": (ctypes.c_char_p, [c_int]),
    "b200_last_cuda_error": (c_int, []),
    "b200_abi_version": (c_int, []),
    "b200_set_sm_limit": (c_int, [c_int]),
    "b200_per_token_group_quant_fp8": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                               c_int64, c_int64, c_float, c_float, c_float, c_void_p]),
    "b200_per_token_group_quant_int8": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                                c_int64, c_int64, c_float, c_float, c_float, c_void_p]),
    "b200_per_token_group_quant_fp8_ieee_div": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64,
                                                        c_int64, c_int64, c_int64, c_float, c_float, c_float,
                                                        c_void_p]),
    "b200_silu_mul_per_token_group_quant_fp8": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                                        c_int64, c_float, c_float, c_float, c_void_p]),
    "b200_per_token_group_quant_fp8_ue8m0": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                                     c_float, c_float, c_float, c_void_p]),
    "b200_fp8_blockwise_scaled_mm": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                             c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int, c_int64, c_int64,
                                             c_int64, c_void_p]),
    "b200_fp8_blockwise_scaled_mm_splitk": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                                    c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int, c_int64,
                                                    c_int64, c_int64, c_int, c_void_p, ctypes.c_size_t, c_void_p]),
    "b200_fp8_blockwise_scaled_mm_splitk_plan": (c_int, [c_int64, c_int64, c_int64, c_int, ctypes.POINTER(c_int),
                                                         ctypes.POINTER(ctypes.c_size_t)]),
    "b200_fp8_blockwise_scaled_mm_ue8m0": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                                   c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int, c_int64,
                                                   c_int64, c_int64, c_void_p]),
    "b200_fp8_blockwise_scaled_mm_pow2": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                                  c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int, c_int64,
                                                  c_int64, c_int64, c_void_p]),
    "b200_fp8_blockwise_scaled_grouped_mm_pow2": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                                          c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                                                          c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64,
                                                          c_void_p, c_int, c_int, c_int64, c_int64, c_void_p]),
    "b200_fp8_blockwise_scaled_grouped_mm_pow2_silu_quant": (c_int, [
        c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64,
        c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int,
        c_int64, c_int64, c_void_p]),
    "b200_silu_mul_per_token_group_quant_fp8_ue8m0": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64,
                                                              c_int64, c_float, c_float, c_float, c_void_p]),
    "b200_gather_per_token_group_quant_fp8": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int64,
                                                      c_int64, c_int64, c_int64, c_int, c_float, c_float, c_float,
                                                      c_void_p]),
    "b200_rmsnorm_per_token_group_quant_fp8": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                                       c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_float,
                                                       c_float, c_float, c_void_p]),
    "b200_per_token_group_quant_fp8_ue8m0_strided": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                                             c_int64, c_float, c_float, c_float, c_void_p]),
    "b200_gemm_device_status": (c_int, [ctypes.POINTER(c_int)]),
    "b200_gemm_poll_status": (c_int, [ctypes.POINTER(c_int)]),
    "b200_fp8_blockwise_scaled_grouped_mm": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                                     c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int,
                                                     c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p]),
    "b200_moe_prepare_scratch_bytes": (ctypes.c_size_t, [c_int64, c_int]),
    "b200_moe_prepare": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_void_p]),
    "b200_moe_prepare_noalloc": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200_moe_align_block_size_scratch_bytes": (ctypes.c_size_t, [c_int64, c_int]),
    "b200_moe_align_block_size": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p, c_int64,
                                          c_void_p, c_void_p, c_int, c_void_p, ctypes.c_size_t, c_void_p]),
    "b200_topk_softmax": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "b200_moe_fused_gate": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                                    c_void_p]),
    "b200_moe_fused_gate_shared_experts": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                                   c_int, c_int, c_int, ctypes.c_double, c_void_p]),
    "b200_shuffle_packed_scales": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int,
                                           c_void_p]),
    "b200_shuffle_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "b200_silu_and_mul": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "b200_apply_shuffle_mul_sum": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                                           c_void_p]),
    "b200_allreduce": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int,
                               c_int, c_int, c_int, c_int64, c_void_p]),
    "b200_allreduce_flag_words": (c_int, [c_int]),
    "b200_allreduce_max_blocks": (c_int, []),
    "b200_ep_buffer_bytes": (c_int64, [c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_ep_dispatch": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                 c_int, c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200_ep_received_expert_ids": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200_ep_combine": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                c_int64, c_void_p, c_void_p, c_void_p]),
    "b200_debug_force_block_n": (c_int, [c_int]),
}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m sglang_b200.build` "
                "(nvcc, sm_100a). There is no fallback implementation.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(fn_name: str, code: int) -> None:
    if code == 0:
        return
    L = lib()
    detail = L.b200_strerror(code).decode()
    if code == -7:
        detail += f" [cudaError {L.b200_last_cuda_error()}]"
    raise B200Error(fn_name, code, detail)


def exported_symbols():
    return list(_SIGNATURES.keys())

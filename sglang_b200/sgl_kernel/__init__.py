"""Drop-in for the block-FP8 subset of the reference's `sgl_kernel` package.

Importing this module registers the operators under torch.ops.sgl_kernel with the reference's
schemas verbatim (sgl-kernel/csrc/common_extension.cc:111-124,165-179,192-207), implemented for the
CUDA dispatch key by the B200 C-ABI library, and exposes the same-named Python wrappers
(sgl-kernel/python/sgl_kernel/{gemm,moe}.py).
"""
import torch

from .gemm import fp8_blockwise_scaled_mm, sgl_per_token_group_quant_fp8, sgl_per_token_group_quant_int8
from .moe import (apply_shuffle_mul_sum, fp8_blockwise_scaled_grouped_mm, prepare_moe_input, shuffle_rows,
                  shuffle_rows_into, shuffle_packed_scales, silu_and_mul, topk_softmax, moe_fused_gate,
                  moe_align_block_size)

_SCHEMAS = {
    "fp8_blockwise_scaled_mm":
        "(Tensor mat_a, Tensor mat_b, Tensor scales_a, Tensor scales_b, ScalarType out_dtype) -> Tensor",
    "sgl_per_token_group_quant_fp8":
        "(Tensor input, Tensor output_q, Tensor output_s, int group_size, float eps, float fp8_min, "
        "float fp8_max, bool scale_ue8m0) -> ()",
    "sgl_per_token_group_quant_int8":
        "(Tensor input, Tensor output_q, Tensor output_s, int group_size, float eps, float int8_min, "
        "float int8_max) -> ()",
    "fp8_blockwise_scaled_grouped_mm":
        "(Tensor output, Tensor a_ptrs, Tensor b_ptrs, Tensor out_ptrs, Tensor a_scales_ptrs, Tensor b_scales_ptrs, "
        "Tensor a, Tensor b, Tensor scales_a, Tensor scales_b, Tensor stride_a, Tensor stride_b, Tensor stride_c, "
        "Tensor layout_sfa, Tensor layout_sfb, Tensor problem_sizes, Tensor expert_offsets, Tensor workspace) -> ()",
    "prepare_moe_input":
        "(Tensor topk_ids, Tensor expert_offsets, Tensor? blockscale_offsets, Tensor problem_sizes1, "
        "Tensor problem_sizes2, Tensor input_permutation, Tensor output_permutation, int num_experts, int n, int k) -> ()",
    "shuffle_rows": "(Tensor input, Tensor dst2src_map, Tensor output) -> ()",
    "apply_shuffle_mul_sum": "(Tensor input, Tensor output, Tensor permutation, Tensor? factors) -> ()",
    "silu_and_mul": "(Tensor out, Tensor input) -> ()",
    "topk_softmax": "(Tensor! topk_weights, Tensor! topk_indices, Tensor gating_output, bool renormalize) -> ()",
    "moe_fused_gate":
        "(Tensor input, Tensor bias, int num_expert_group, int topk_group, int topk, int num_fused_shared_experts, "
        "float routed_scaling_factor) -> (Tensor[])",
    "moe_align_block_size":
        "(Tensor topk_ids, int num_experts, int block_size, Tensor! sorted_token_ids, Tensor! experts_ids, "
        "Tensor! num_tokens_post_pad, Tensor! cumsum_buffer, bool pad_sorted_token_ids) -> ()",
}


def _prepare_moe_input_op(topk_ids, expert_offsets, blockscale_offsets, problem_sizes1, problem_sizes2,
                          input_permutation, output_permutation, num_experts, n, k):
    prepare_moe_input(topk_ids, expert_offsets, problem_sizes1, problem_sizes2, input_permutation,
                      output_permutation, num_experts, n, k, blockscale_offsets)


def _silu_and_mul_op(out, input):
    silu_and_mul(input, out)


def _moe_fused_gate_op(input, bias, num_expert_group, topk_group, topk, num_fused_shared_experts, routed_scaling_factor):
    return list(moe_fused_gate(input, bias, num_expert_group, topk_group, topk, num_fused_shared_experts,
                               routed_scaling_factor))


def _moe_fused_gate_meta(input, bias, num_expert_group, topk_group, topk, num_fused_shared_experts, routed_scaling_factor):
    return [input.new_empty((input.shape[0], topk), dtype=torch.float32),
            input.new_empty((input.shape[0], topk), dtype=torch.int32)]


_IMPLS = {
    "fp8_blockwise_scaled_mm": fp8_blockwise_scaled_mm,
    "sgl_per_token_group_quant_fp8": sgl_per_token_group_quant_fp8,
    "sgl_per_token_group_quant_int8": sgl_per_token_group_quant_int8,
    "fp8_blockwise_scaled_grouped_mm": fp8_blockwise_scaled_grouped_mm,
    "prepare_moe_input": _prepare_moe_input_op,
    "shuffle_rows": shuffle_rows_into,
    "apply_shuffle_mul_sum": apply_shuffle_mul_sum,
    "silu_and_mul": _silu_and_mul_op,
    "topk_softmax": topk_softmax,
    "moe_align_block_size": moe_align_block_size,
    "moe_fused_gate": _moe_fused_gate_op,
}



def _mm_meta(mat_a, mat_b, scales_a, scales_b, out_dtype):
    return mat_a.new_empty((mat_a.shape[0], mat_b.shape[1]), dtype=out_dtype)


def _nothing_meta(*args):
    return None


# Shape functions for tracing (meta tensors / fake tensors): only the dense GEMM returns a tensor; the
# other operators write into tensors the caller allocated.
_META = {name: _nothing_meta for name in _SCHEMAS}
_META["fp8_blockwise_scaled_mm"] = _mm_meta
_META["moe_fused_gate"] = _moe_fused_gate_meta

_library = None


def register_torch_ops() -> None:
    """Idempotent; skipped for operators another package (the real sgl_kernel) already defined."""
    global _library
    if _library is not None:
        return
    _library = torch.library.Library("sgl_kernel", "FRAGMENT")
    for name, schema in _SCHEMAS.items():
        try:
            _library.define(name + schema)
        except RuntimeError:
            continue  # already defined elsewhere: leave that definition alone
        _library.impl(name, _IMPLS[name], "CUDA")
        _library.impl(name, _META[name], "Meta")


register_torch_ops()

__all__ = ["fp8_blockwise_scaled_mm", "sgl_per_token_group_quant_fp8", "sgl_per_token_group_quant_int8", "fp8_blockwise_scaled_grouped_mm",
           "prepare_moe_input", "shuffle_rows", "shuffle_packed_scales", "apply_shuffle_mul_sum", "silu_and_mul", "topk_softmax",
           "moe_fused_gate", "moe_align_block_size", "register_torch_ops"]

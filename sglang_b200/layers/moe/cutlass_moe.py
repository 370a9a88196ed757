"""Fused MoE with block-FP8 experts: the op sequence of the reference's
`cutlass_fused_experts_fp8` (python/sglang/srt/layers/moe/cutlass_moe.py:29-222), same signature.

prepare_moe_input -> group quant -> row gather -> grouped GEMM 1 -> SiLU*mul -> group quant ->
grouped GEMM 2 -> weighted un-permute sum.  Nothing on the host looks at device data (routing
counts stay on the device), so the whole sequence is stream-ordered.
"""
from __future__ import annotations

from typing import Optional

import torch

from ...sgl_kernel import (apply_shuffle_mul_sum, fp8_blockwise_scaled_grouped_mm, prepare_moe_input,
                           shuffle_packed_scales, shuffle_rows, silu_and_mul)
from ..quantization.deep_gemm_wrapper import grouped_gemm_pow2, grouped_gemm_pow2_silu_quant
from ..quantization.fp8_kernel import sglang_per_token_group_quant_fp8, silu_and_mul_per_token_group_quant_fp8


def cutlass_fused_experts_fp8(
    a: torch.Tensor,
    w1_q: torch.Tensor,
    w2_q: torch.Tensor,
    w1_scale: torch.Tensor,
    w2_scale: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    a1_strides: Optional[torch.Tensor] = None,
    c1_strides: Optional[torch.Tensor] = None,
    a2_strides: Optional[torch.Tensor] = None,
    c2_strides: Optional[torch.Tensor] = None,
    workspace: Optional[torch.Tensor] = None,
    a_ptrs: Optional[torch.Tensor] = None,
    b_ptrs: Optional[torch.Tensor] = None,
    out_ptrs: Optional[torch.Tensor] = None,
    a_scales_ptrs: Optional[torch.Tensor] = None,
    b_scales_ptrs: Optional[torch.Tensor] = None,
    expert_offsets: Optional[torch.Tensor] = None,
    problem_sizes1: Optional[torch.Tensor] = None,
    problem_sizes2: Optional[torch.Tensor] = None,
    use_fp8_blockscale: bool = True,
) -> torch.Tensor:
    """a [m, k] bf16/fp16; w1_q [E, k, 2n] and w2_q [E, n, k] e4m3 (transposed views of the
    [E, N, K] weights, as the reference passes them); w1_scale / w2_scale: block scales whose memory
    order is [E][N/128][K/128]; topk_weights / topk_ids [m, topk] (ids int32).  The stride, pointer
    and workspace tensors are scratch of the reference kernels: accepted, not needed.  The three
    routing tensors are allocated here when not supplied.  Returns [m, k] in a.dtype."""
    assert use_fp8_blockscale, "Only support fp8 blockscale for now"
    assert topk_weights.shape == topk_ids.shape, "topk shape mismatch"
    assert w1_q.dtype == torch.float8_e4m3fn
    assert w2_q.dtype == torch.float8_e4m3fn
    assert a.shape[1] == w1_q.shape[1], "Hidden size mismatch w1"
    assert w1_q.shape[2] == w2_q.shape[1] * 2, "Hidden size mismatch w2"
    assert w1_q.shape[0] == w2_q.shape[0], "Expert number mismatch"
    assert w1_q.shape[0] == w1_scale.shape[0], "w1 scales expert number mismatch"
    assert w1_q.shape[0] == w2_scale.shape[0], "w2 scales expert number mismatch"
    assert a.dtype in [torch.half, torch.bfloat16], "Invalid output dtype"

    out_dtype = a.dtype
    num_experts = w1_q.size(0)
    m = a.size(0)
    k = w1_q.size(1)
    n = w2_q.size(1)
    topk = topk_ids.size(1)
    device = a.device
    i32 = dict(dtype=torch.int32, device=device)
    if expert_offsets is None:
        expert_offsets = torch.empty(num_experts + 1, **i32)
    if problem_sizes1 is None:
        problem_sizes1 = torch.empty((num_experts, 3), **i32)
    if problem_sizes2 is None:
        problem_sizes2 = torch.empty((num_experts, 3), **i32)
    topk_ids = topk_ids.to(torch.int32).contiguous()

    a_map = torch.zeros((topk_ids.numel()), **i32)   # unrouted slots gather row 0 (in bounds, never used)
    c_map = torch.empty((topk_ids.numel()), **i32)
    prepare_moe_input(topk_ids, expert_offsets, problem_sizes1, problem_sizes2, a_map, c_map, num_experts, n, k)

    a_q, a1_scale = sglang_per_token_group_quant_fp8(a, 128)
    rep_a_q = shuffle_rows(a_q, a_map, (m * topk, k))
    rep_a1_scales = shuffle_rows(a1_scale, a_map, (m * topk, int(k / 128)))

    c1 = torch.empty((m * topk, n * 2), device=device, dtype=out_dtype)
    c2 = torch.empty((m * topk, k), device=device, dtype=out_dtype)
    fp8_blockwise_scaled_grouped_mm(c1, a_ptrs, b_ptrs, out_ptrs, a_scales_ptrs, b_scales_ptrs, rep_a_q, w1_q,
                                    rep_a1_scales, w1_scale, a1_strides, a1_strides, c1_strides, None, None,
                                    problem_sizes1, expert_offsets[:-1], workspace)

    # SiLU*mul and the second group quantisation in one pass (bit-identical to the two-kernel sequence
    # silu_and_mul -> sglang_per_token_group_quant_fp8 of the reference, cutlass_moe.py:191-194)
    intermediate_q, a2_scale = silu_and_mul_per_token_group_quant_fp8(c1, 128)
    fp8_blockwise_scaled_grouped_mm(c2, a_ptrs, b_ptrs, out_ptrs, a_scales_ptrs, b_scales_ptrs, intermediate_q, w2_q,
                                    a2_scale, w2_scale, a2_strides, a2_strides, c2_strides, None, None,
                                    problem_sizes2, expert_offsets[:-1], workspace)

    result = torch.empty((m, k), device=device, dtype=out_dtype)
    apply_shuffle_mul_sum(c2, result, c_map, topk_weights.to(out_dtype))
    return result


def fused_experts_block_fp8(a, w13, w2, w13_scale, w2_scale, topk_weights, topk_ids):
    """Convenience form with natural weight layouts: w13 [E, 2n, k], w2 [E, k, n] e4m3 contiguous,
    scales [E, 2n/128, k/128] and [E, k/128, n/128] -- what Fp8MoEMethod holds
    (python/sglang/srt/layers/quantization/fp8.py:1030-1065 passes the transposed views)."""
    return cutlass_fused_experts_fp8(a, w13.transpose(1, 2), w2.transpose(1, 2), w13_scale.transpose(1, 2),
                                     w2_scale.transpose(1, 2), topk_weights, topk_ids)


def fused_experts_block_fp8_ue8m0(a, w13, w2, w13_scale, w2_scale, topk_weights, topk_ids,
                                  fuse_activation: bool = True):
    """The fused expert layer on the tensor core's block-scaling path: activations quantised to power-of-two
    scales, weights w13 [E, 2n, k] / w2 [E, k, n] e4m3 with POWER-OF-TWO fp32 block scales [E, 2n/128, k/128] /
    [E, k/128, n/128] (requant_weight_ue8m0 at load time).  The reference's counterpart is its DeepGEMM expert path
    with UE8M0 scales (python/sglang/srt/layers/moe/ep_moe/layer.py:540-640: scatter -> contiguous grouped GEMM ->
    SiLU*mul -> quant -> grouped GEMM -> weighted gather); here every expert's rows are packed without padding and
    the schedule reads offsets and counts on the device.  fuse_activation: SiLU*mul and the second quantisation run in
    the first GEMM's epilogue (same bits as the separate kernels)."""
    assert topk_weights.shape == topk_ids.shape
    assert a.dtype in (torch.half, torch.bfloat16) and a.dim() == 2 and a.is_contiguous()
    E, n2, k = w13.shape
    n = w2.shape[2]
    assert n2 == 2 * n and w2.shape == (E, k, n) and a.shape[1] == k
    m, topk = topk_ids.shape
    device = a.device
    i32 = dict(dtype=torch.int32, device=device)
    expert_offsets = torch.empty(E + 1, **i32)
    ps1, ps2 = torch.empty((E, 3), **i32), torch.empty((E, 3), **i32)
    ids = topk_ids.to(torch.int32).contiguous()
    a_map = torch.zeros(ids.numel(), **i32)      # unrouted slots gather row 0 (in bounds, never used)
    c_map = torch.empty(ids.numel(), **i32)
    prepare_moe_input(ids, expert_offsets, ps1, ps2, a_map, c_map, E, n, k)
    # every token is quantised once; its codes and packed scale words are then copied to the rows of its experts
    # (quantising after the copy would do the arithmetic topk times: measured 189 us against 95 us for this size)
    a_q, a_s = sglang_per_token_group_quant_fp8(a, 128, column_major_scales=True, scale_tma_aligned=True,
                                                scale_ue8m0=True)
    rep_q = shuffle_rows(a_q, a_map, (m * topk, k))
    rep_s = shuffle_packed_scales(a_s, a_map)
    rows = ps1[:, 0]
    if fuse_activation:
        # GEMM 1 with SiLU*mul and GEMM 2's quantisation in its epilogue: the [rows, 2n] intermediate stays on chip
        inter_q, inter_s = grouped_gemm_pow2_silu_quant(rep_q, rep_s, w13, w13_scale, expert_offsets[:-1], rows,
                                                        mid_dtype=a.dtype)
    else:
        c1 = torch.empty((m * topk, 2 * n), device=device, dtype=a.dtype)
        grouped_gemm_pow2(rep_q, rep_s, w13, w13_scale, c1, expert_offsets[:-1], rows)
        inter_q, inter_s = silu_and_mul_per_token_group_quant_fp8(c1, 128, scale_ue8m0=True)
    c2 = torch.empty((m * topk, k), device=device, dtype=a.dtype)
    grouped_gemm_pow2(inter_q, inter_s, w2, w2_scale, c2, expert_offsets[:-1], rows)
    result = torch.empty((m, k), device=device, dtype=a.dtype)
    apply_shuffle_mul_sum(c2, result, c_map, topk_weights.to(a.dtype))
    return result


def grouped_experts_prequantized(a_q, a_scale, expert_ids, w13, w2, w13_scale, w2_scale, out_dtype=torch.bfloat16,
                                 return_sorted: bool = False):
    """Expert MLPs over rows that are ALREADY quantised (what an expert-parallel rank receives):
    a_q [R, k] e4m3, a_scale [R, k/128] fp32, expert_ids [R] int32 (local ids; < 0 = skip).
    Returns [R, k] in out_dtype, rows in input order, no routing weights applied; with `return_sorted` the
    rows stay grouped by expert and the second result maps input row -> its row there (skipped rows map
    nowhere meaningful), which saves one pass when the caller scatters the rows anyway."""
    R, k = a_q.shape
    E, n = w13.shape[0], w2.shape[2]
    device = a_q.device
    i32 = dict(dtype=torch.int32, device=device)
    ids = expert_ids.to(torch.int32).reshape(R, 1).contiguous()
    expert_offsets = torch.empty(E + 1, **i32)
    ps1, ps2 = torch.empty((E, 3), **i32), torch.empty((E, 3), **i32)
    a_map, c_map = torch.zeros(R, **i32), torch.empty(R, **i32)
    prepare_moe_input(ids, expert_offsets, ps1, ps2, a_map, c_map, E, n, k)
    rep_q = shuffle_rows(a_q, a_map, (R, k))
    rep_s = shuffle_rows(a_scale.contiguous(), a_map, (R, k // 128))
    c1 = torch.empty((R, 2 * n), device=device, dtype=out_dtype)
    fp8_blockwise_scaled_grouped_mm(c1, None, None, None, None, None, rep_q, w13.transpose(1, 2), rep_s,
                                    w13_scale, None, None, None, None, None, ps1, expert_offsets[:-1], None)
    inter_q, inter_s = silu_and_mul_per_token_group_quant_fp8(c1, 128)
    c2 = torch.empty((R, k), device=device, dtype=out_dtype)
    fp8_blockwise_scaled_grouped_mm(c2, None, None, None, None, None, inter_q, w2.transpose(1, 2), inter_s,
                                    w2_scale, None, None, None, None, None, ps2, expert_offsets[:-1], None)
    if return_sorted:
        return c2, c_map
    out = torch.empty((R, k), device=device, dtype=out_dtype)
    apply_shuffle_mul_sum(c2, out, c_map, None)     # topk = 1: pure un-permute back to input order
    return out


def grouped_experts_prequantized_ue8m0(a_q, a_words, expert_ids, w13, w2, w13_scale, w2_scale,
                                       out_dtype=torch.bfloat16, return_sorted: bool = False):
    """grouped_experts_prequantized on the block-scaling path: a_q [R, k] e4m3, a_words [R, W] int32 -- each row's
    packed power-of-two exponents, contiguous per row (per_token_group_quant_fp8_ue8m0_rows) -- expert_ids [R] int32
    (< 0 = skip); weights with power-of-two block scales."""
    R, k = a_q.shape
    E, n = w13.shape[0], w2.shape[2]
    device = a_q.device
    i32 = dict(dtype=torch.int32, device=device)
    ids = expert_ids.to(torch.int32).reshape(R, 1).contiguous()
    expert_offsets = torch.empty(E + 1, **i32)
    ps1, ps2 = torch.empty((E, 3), **i32), torch.empty((E, 3), **i32)
    a_map, c_map = torch.zeros(R, **i32), torch.empty(R, **i32)
    prepare_moe_input(ids, expert_offsets, ps1, ps2, a_map, c_map, E, n, k)
    rep_q = shuffle_rows(a_q, a_map, (R, k))
    rep_w = shuffle_rows(a_words.contiguous(), a_map, (R, a_words.shape[1]))       # rows of words: a plain row gather
    rows = ps1[:, 0]
    inter_q, inter_s = grouped_gemm_pow2_silu_quant(rep_q, rep_w, w13, w13_scale, expert_offsets[:-1], rows,
                                                    mid_dtype=out_dtype)
    c2 = torch.empty((R, k), device=device, dtype=out_dtype)
    grouped_gemm_pow2(inter_q, inter_s, w2, w2_scale, c2, expert_offsets[:-1], rows)
    if return_sorted:
        return c2, c_map
    out = torch.empty((R, k), device=device, dtype=out_dtype)
    apply_shuffle_mul_sum(c2, out, c_map, None)
    return out

"""Python surface of the reference's `sgl_kernel.moe` / `sgl_kernel.gemm.shuffle_rows` /
`sgl_kernel.elementwise.silu_and_mul` for the block-FP8 MoE path, backed by the B200 C-ABI library.

Mirrors (names, argument order, error behaviour):
  prepare_moe_input                 sgl-kernel/python/sgl_kernel/moe.py:173-196
  fp8_blockwise_scaled_grouped_mm   sgl-kernel/python/sgl_kernel/moe.py:131-170
  apply_shuffle_mul_sum             sgl-kernel/python/sgl_kernel/moe.py:199-207
  shuffle_rows                      sgl-kernel/python/sgl_kernel/gemm.py:281-288
  silu_and_mul                      sgl-kernel/python/sgl_kernel/elementwise.py:171-183
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib
from .gemm import _DT, FP8, _check, _stream_ptr


def topk_softmax(topk_weights: torch.Tensor, topk_ids: torch.Tensor, gating_output: torch.Tensor,
                 renormalize: bool = False) -> None:
    """In place: topk_weights [m, k] fp32 <- the k largest softmax probabilities of each row of
    gating_output [m, E] (fp32 / fp16 / bf16), topk_ids [m, k] int32 <- their expert ids.
    Mirrors sgl_kernel.topk_softmax (sgl-kernel/python/sgl_kernel/moe.py:28-36) and the checks of its C++ entry
    (sgl-kernel/csrc/moe/moe_topk_softmax_kernels.cu:508-529)."""
    _check(gating_output.dtype in _DT, "gating_output must be float32, float16, or bfloat16")
    _check(gating_output.dim() == 2, "gating_output must be 2D tensor [num_tokens, num_experts]")
    _check(topk_weights.dim() == 2, "topk_weights must be 2D tensor [num_tokens, topk]")
    _check(topk_ids.dim() == 2, "topk_indices must be 2D tensor [num_tokens, topk]")
    _check(gating_output.size(0) == topk_weights.size(0),
           "First dimension of topk_weights must match num_tokens in gating_output")
    _check(gating_output.size(0) == topk_ids.size(0),
           "First dimension of topk_indices must match num_tokens in gating_output")
    _check(topk_weights.size(-1) == topk_ids.size(-1), "Second dimension of topk_indices must match topk in topk_weights")
    _check(topk_weights.size(-1) <= gating_output.size(-1), "topk must be less than or equal to num_experts")
    _check(gating_output.is_cuda and topk_weights.is_cuda and topk_ids.is_cuda, "tensors must be CUDA tensors")
    _check(topk_weights.dtype == torch.float32 and topk_weights.is_contiguous(), "topk_weights must be contiguous float32")
    _check(topk_ids.dtype == torch.int32 and topk_ids.is_contiguous(), "topk_indices must be contiguous int32")
    _check(gating_output.stride(1) == 1, "gating_output rows must be contiguous")
    m, E = gating_output.shape
    with torch.cuda.device(gating_output.device):
        rc = _lib.lib().b200_topk_softmax(gating_output.data_ptr(), _DT[gating_output.dtype], gating_output.stride(0),
                                          topk_weights.data_ptr(), topk_ids.data_ptr(), m, E, topk_weights.size(1),
                                          int(bool(renormalize)), _stream_ptr(gating_output.device))
    _lib.check("topk_softmax", rc)


def moe_align_block_size(topk_ids: torch.Tensor, num_experts: int, block_size: int, sorted_token_ids: torch.Tensor,
                         experts_ids: torch.Tensor, num_tokens_post_pad: torch.Tensor, cumsum_buffer: torch.Tensor,
                         pad_sorted_token_ids: bool = False) -> None:
    """In place: the flat indices of topk_ids grouped by expert into sorted_token_ids, every expert's run padded
    to a multiple of block_size; experts_ids <- the expert of each block; num_tokens_post_pad <- padded length.
    `num_experts` counts the slots (experts + 1, slot 0 = id -1) as in the reference.  Mirrors
    sgl_kernel.moe_align_block_size (sgl-kernel/python/sgl_kernel/moe.py:6-25; kernel
    sgl-kernel/csrc/moe/moe_align_kernel.cu:283-366).  Inside an expert the indices ascend."""
    _check(topk_ids.is_cuda and sorted_token_ids.is_cuda and experts_ids.is_cuda and num_tokens_post_pad.is_cuda
           and cumsum_buffer.is_cuda, "tensors must be CUDA tensors")
    _check(topk_ids.dtype in (torch.int32, torch.int64) and topk_ids.is_contiguous(),
           "topk_ids must be contiguous int32 or int64")
    for name, t in (("sorted_token_ids", sorted_token_ids), ("experts_ids", experts_ids),
                    ("num_tokens_post_pad", num_tokens_post_pad), ("cumsum_buffer", cumsum_buffer)):
        _check(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be contiguous int32")
    _check(num_tokens_post_pad.numel() >= 1, "num_tokens_post_pad must hold one element")
    _check(cumsum_buffer.numel() >= num_experts + 1, "cumsum_buffer must hold num_experts + 1 elements")
    numel = topk_ids.numel()
    lib = _lib.lib()
    need = lib.b200_moe_align_block_size_scratch_bytes(numel, num_experts)
    scratch = torch.empty((max(need, 4) // 4,), dtype=torch.int32, device=topk_ids.device) if need else None
    with torch.cuda.device(topk_ids.device):
        rc = lib.b200_moe_align_block_size(topk_ids.data_ptr(), int(topk_ids.dtype == torch.int64), numel, num_experts,
                                           block_size, sorted_token_ids.data_ptr(), sorted_token_ids.numel(),
                                           experts_ids.data_ptr(), experts_ids.numel(), num_tokens_post_pad.data_ptr(),
                                           cumsum_buffer.data_ptr(), int(bool(pad_sorted_token_ids)),
                                           scratch.data_ptr() if scratch is not None else None, need,
                                           _stream_ptr(topk_ids.device))
    _lib.check("moe_align_block_size", rc)


def moe_fused_gate(input_tensor: torch.Tensor, bias: torch.Tensor, num_expert_group: int, topk_group: int, topk: int,
                   num_fused_shared_experts: int = 0, routed_scaling_factor: float = 0):
    """DeepSeek-V3 gate (sigmoid scores, choice bias, group-limited top-k, weights renormalised): returns
    (topk_weights fp32 [m, k], topk_ids int32 [m, k]).  Mirrors sgl_kernel.moe_fused_gate
    (sgl-kernel/python/sgl_kernel/moe.py:39-66).  With num_fused_shared_experts > 0 the last that many of the
    topk slots are the fused shared experts: ids num_experts, num_experts + 1, ..., weight
    1 / routed_scaling_factor; the routed slots before them are renormalised over themselves
    (sgl-kernel/csrc/moe/moe_fused_gate.cu:225-252)."""
    _check(0 <= num_fused_shared_experts < topk, "num_fused_shared_experts must be smaller than topk")
    _check(num_fused_shared_experts == 0 or routed_scaling_factor != 0, "routed_scaling_factor must be non-zero")
    _check(input_tensor.is_cuda and bias.is_cuda, "tensors must be CUDA tensors")
    _check(input_tensor.dim() == 2 and bias.dim() == 1 and bias.numel() == input_tensor.size(1), "shape mismatch")
    _check(input_tensor.dtype == torch.float32 and bias.dtype == torch.float32, "input and bias must be float32")
    _check(input_tensor.stride(1) == 1 and bias.is_contiguous(), "rows must be contiguous")
    m, E = input_tensor.shape
    _check(E % num_expert_group == 0 and num_expert_group <= 32 and E // num_expert_group >= 2 and E <= 1024,
           "unsupported expert grouping")
    _check(0 < topk_group <= num_expert_group and topk <= 32 and
           0 < topk - num_fused_shared_experts <= topk_group * (E // num_expert_group), "unsupported topk / topk_group")
    weights = torch.empty((m, topk), dtype=torch.float32, device=input_tensor.device)
    ids = torch.empty((m, topk), dtype=torch.int32, device=input_tensor.device)
    with torch.cuda.device(input_tensor.device):
        rc = _lib.lib().b200_moe_fused_gate_shared_experts(
            input_tensor.data_ptr(), input_tensor.stride(0), bias.data_ptr(), weights.data_ptr(), ids.data_ptr(), m, E,
            num_expert_group, topk_group, topk, int(num_fused_shared_experts),
            float(routed_scaling_factor) if num_fused_shared_experts else 1.0, _stream_ptr(input_tensor.device))
    _lib.check("moe_fused_gate", rc)
    return weights, ids


def prepare_moe_input(topk_ids, expert_offsets, problem_sizes1, problem_sizes2, input_permutation,
                      output_permutation, num_experts, n, k, blockscale_offsets: Optional[torch.Tensor] = None):
    """In place.  topk_ids [m, topk] int32; expert_offsets [E+1]; problem_sizes* [E,3];
    permutations [m*topk] int32.  The scratch table this op needs is allocated here, the way the
    reference allocates its atomic buffer (prepare_moe_input.cu:106)."""
    _check(topk_ids.dtype == torch.int32, "topk_ids must be int32")
    _check(topk_ids.is_cuda and topk_ids.is_contiguous(), "topk_ids must be a contiguous CUDA tensor")
    for t in (expert_offsets, problem_sizes1, problem_sizes2, input_permutation, output_permutation):
        _check(t.dtype == torch.int32 and t.is_cuda and t.is_contiguous(), "index tensors must be contiguous int32 CUDA")
    _check(expert_offsets.numel() >= num_experts + 1, "expert_offsets must hold num_experts + 1 entries")
    _check(problem_sizes1.numel() >= 3 * num_experts and problem_sizes2.numel() >= 3 * num_experts,
           "problem_sizes must be [num_experts, 3]")
    _check(input_permutation.numel() >= topk_ids.numel() and output_permutation.numel() >= topk_ids.numel(),
           "permutations must hold topk_ids.numel() entries")
    m, topk = topk_ids.shape
    L = _lib.lib()
    nbytes = L.b200_moe_prepare_scratch_bytes(topk_ids.numel(), num_experts)
    scratch = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=topk_ids.device)
    with torch.cuda.device(topk_ids.device):
        rc = L.b200_moe_prepare(topk_ids.data_ptr(), m, topk, num_experts, n, k, expert_offsets.data_ptr(),
                                blockscale_offsets.data_ptr() if blockscale_offsets is not None else None,
                                problem_sizes1.data_ptr(), problem_sizes2.data_ptr(), input_permutation.data_ptr(),
                                output_permutation.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                _stream_ptr(topk_ids.device))
    _lib.check("prepare_moe_input", rc)


def shuffle_rows_into(input_tensor: torch.Tensor, dst2src_map: torch.Tensor, output_tensor: torch.Tensor) -> None:
    """The op itself (schema `shuffle_rows(Tensor input, Tensor dst2src_map, Tensor output) -> ()`)."""
    _check(input_tensor.dtype == output_tensor.dtype, "Input and output tensors must have the same data type")
    _check(input_tensor.is_cuda and input_tensor.is_contiguous() and output_tensor.is_contiguous(),
           "tensors must be contiguous CUDA tensors")
    _check(dst2src_map.dtype == torch.int32, "dst2src_map must be int32")
    _check(input_tensor.dim() == 2 and output_tensor.dim() == 2 and input_tensor.size(1) == output_tensor.size(1),
           "row length mismatch")
    row_bytes = input_tensor.size(1) * input_tensor.element_size()
    with torch.cuda.device(input_tensor.device):
        rc = _lib.lib().b200_shuffle_rows(input_tensor.data_ptr(), dst2src_map.data_ptr(), output_tensor.data_ptr(),
                                          output_tensor.size(0), row_bytes, _stream_ptr(input_tensor.device))
    _lib.check("shuffle_rows", rc)


def shuffle_rows(input_tensor, dst2src_map, output_tensor_shape):
    output_tensor = torch.empty(output_tensor_shape, device=input_tensor.device, dtype=input_tensor.dtype)
    shuffle_rows_into(input_tensor, dst2src_map, output_tensor)
    return output_tensor


def shuffle_packed_scales(packed: torch.Tensor, dst2src_map: torch.Tensor) -> torch.Tensor:
    """Row gather of the packed power-of-two scales that sglang_per_token_group_quant_fp8(scale_ue8m0=True) returns
    (int32 [M, W], rows contiguous): result [R, W] in the same layout with row r = packed[dst2src_map[r]]."""
    _check(packed.dtype == torch.int32 and packed.dim() == 2, "packed scales must be int32 [rows, words]")
    _check(packed.stride(0) == 1 or packed.size(0) == 1, "packed scales must have their rows contiguous")
    _check(dst2src_map.dtype == torch.int32 and dst2src_map.is_contiguous(), "dst2src_map must be int32")
    M, W = packed.shape
    R = dst2src_map.numel()
    aligned = (R + 3) // 4 * 4
    out = torch.zeros((W, aligned), dtype=torch.int32, device=packed.device).transpose(0, 1)[:R, :]
    if R > 0:
        with torch.cuda.device(packed.device):
            rc = _lib.lib().b200_shuffle_packed_scales(packed.data_ptr(), packed.stride(1), M, dst2src_map.data_ptr(),
                                                       out.data_ptr(), out.stride(1), R, W, _stream_ptr(packed.device))
        _lib.check("shuffle_packed_scales", rc)
    return out


def apply_shuffle_mul_sum(input, output, permutation, factors):
    """output[i] = sum_j factors[i,j] * input[permutation[i*topk+j]] (fp32 accumulate)."""
    _check(input.dim() == 2, "input_tensor must be 2D [m * topk, row_stride]")
    _check(output.dim() == 2, "output_tensor must be 2D [m, row_stride]")
    _check(permutation.dim() == 1, "permutation must be 1D [m * topk]")
    m = output.size(0)
    if m == 0:
        return
    topk = permutation.size(0) // m
    _check(permutation.size(0) == m * topk, "permutation size must match m * topk")
    _check(permutation.dtype == torch.int32, "permutation must be int32")
    _check(input.dtype == output.dtype and input.dtype in (torch.bfloat16, torch.float16),
           "input/output must be bfloat16 or float16")
    fptr = None
    if factors is not None:
        _check(factors.dtype == output.dtype, "Factors must match output dtype")
        _check(factors.numel() == m * topk, "Factors must have shape [m * topk]")
        factors = factors.contiguous()
        fptr = factors.data_ptr()
    _check(input.is_contiguous() and output.is_contiguous(), "tensors must be contiguous")
    _check(input.size(1) == output.size(1), "row length mismatch")
    with torch.cuda.device(input.device):
        rc = _lib.lib().b200_apply_shuffle_mul_sum(input.data_ptr(), output.data_ptr(), permutation.data_ptr(), fptr,
                                                   m, topk, output.size(1), _DT[output.dtype],
                                                   _stream_ptr(input.device))
    _lib.check("apply_shuffle_mul_sum", rc)


def silu_and_mul(input: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    if input.shape[-1] * input.dtype.itemsize % 16 != 0:
        raise ValueError("The pointers must be multiple of 16 bytes.")
    d = input.shape[-1] // 2
    if out is None:
        out = torch.empty(input.shape[:-1] + (d,), device=input.device, dtype=input.dtype)
    else:
        assert out.shape == input.shape[:-1] + (d,)
    _check(input.is_contiguous() and out.is_contiguous(), "tensors must be contiguous")
    _check(input.dtype in (torch.bfloat16, torch.float16), "silu_and_mul: bfloat16 or float16 only")
    rows = input.numel() // (2 * d) if d else 0
    with torch.cuda.device(input.device):
        rc = _lib.lib().b200_silu_and_mul(input.data_ptr(), out.data_ptr(), rows, d, _DT[input.dtype],
                                          _stream_ptr(input.device))
    _lib.check("silu_and_mul", rc)
    return out


def fp8_blockwise_scaled_grouped_mm(output, a_ptrs, b_ptrs, out_ptrs, a_scales_ptrs, b_scales_ptrs, a, b, scales_a,
                                    scales_b, stride_a, stride_b, stride_c, layout_sfa, layout_sfb, problem_sizes,
                                    expert_offsets, workspace):
    """Grouped block-FP8 GEMM, in place into `output` [rows, N].

    a [rows, K] e4m3 (rows grouped by expert); b [E, K, N] = weight[E, N, K].transpose(1, 2);
    scales_a [rows, K/128] fp32 row-major; scales_b: memory order [E][N/128][K/128] (the op reads
    only its data pointer, as the reference does -- sgl-kernel/csrc/moe/cutlass_moe_helper.cu:58,69);
    problem_sizes [E, 3] int32 (m, n, k); expert_offsets [E] int32.  The pointer / stride / layout /
    workspace tensors are the reference kernel's scratch; they are accepted and ignored.
    """
    _check(output.is_cuda and a.is_cuda and b.is_cuda, "tensors must be CUDA tensors")
    _check(a.dim() == 2 and b.dim() == 3 and output.dim() == 2, "a, output must be 2D and b 3D")
    _check(a.dtype == FP8 and b.dtype == FP8, "a and b must be Float8_e4m3fn")
    _check(output.dtype in (torch.bfloat16, torch.float16), "output must be bfloat16 or float16")
    _check(scales_a.dtype == torch.float32 and scales_b.dtype == torch.float32, "scales must be Float32")
    _check(scales_a.dim() == 2 and scales_b.dim() == 3, "scales_a must be 2D and scales_b 3D")
    _check(problem_sizes.dim() == 2 and problem_sizes.size(1) == 3 and problem_sizes.dtype == torch.int32,
           "problem_sizes must be int32 [num_experts, 3]")
    _check(expert_offsets.dtype == torch.int32, "expert_offsets must be int32")
    E, K, N = b.shape
    _check(problem_sizes.size(0) == E and expert_offsets.numel() >= E, "one problem size and offset per expert")
    _check(a.size(1) == K and output.size(1) == N and output.size(0) == a.size(0), "shape mismatch")
    _check(b.stride(1) == 1 and b.stride(2) == K and b.stride(0) == N * K,
           "b must be weight[E, N, K].transpose(1, 2) with contiguous experts")
    _check(a.stride(1) == 1 and output.is_contiguous(), "a must be row major and output contiguous")
    _check(K % 128 == 0 and N % 128 == 0, "K and N must be multiples of 128")
    _check(scales_a.is_contiguous() and scales_a.shape == (a.size(0), K // 128), "scales_a must be row-major [rows, K/128]")
    _check(scales_b.numel() == E * (N // 128) * (K // 128), "scales_b size mismatch")
    _check(problem_sizes.is_contiguous(), "problem_sizes must be contiguous")
    if a.size(0) == 0:
        return
    G = K // 128
    with torch.cuda.device(a.device):
        rc = _lib.lib().b200_fp8_blockwise_scaled_grouped_mm(
            a.data_ptr(), a.stride(0), b.data_ptr(), K, scales_a.data_ptr(), G, 1,
            scales_b.data_ptr(), (N // 128) * G, G, 1, output.data_ptr(), output.stride(0), _DT[output.dtype],
            expert_offsets.data_ptr(), problem_sizes.data_ptr(), E, a.size(0), N, K, _stream_ptr(a.device))
    _lib.check("fp8_blockwise_scaled_grouped_mm", rc)

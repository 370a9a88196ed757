"""Glue of the dense block-FP8 linear, mirroring
python/sglang/srt/layers/quantization/fp8_utils.py:182-212
(cutlass_w8a8_block_fp8_linear_with_fallback): view(-1,K) -> group quant with column-major
scales -> block-scaled GEMM -> += bias -> view back.  There is exactly one backend here, so the
reference's dispatch_w8a8_block_fp8_linear (:137-147) returns this function.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ...sgl_kernel import fp8_blockwise_scaled_mm
from .fp8_kernel import sglang_per_token_group_quant_fp8, w8a8_block_fp8_matmul, w8a8_block_fp8_matmul_deepgemm


def ragged_w8a8_block_fp8_linear(input: torch.Tensor, weight: torch.Tensor, block_size: List[int],
                                 weight_scale: torch.Tensor, input_scale: Optional[torch.Tensor] = None,
                                 bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Weights whose N or K is not a multiple of 128 (DeepSeek-V3's kv_a_proj_with_mqa has N = 576) with
    ceil-sized block scales: row-major activation scales and the [N, K]-weight entry of the same CUDA kernel,
    which masks the ragged last block.  Takes the place of the reference's triton_w8a8_block_fp8_linear
    (python/sglang/srt/layers/quantization/fp8_utils.py:289-309), the branch its CUTLASS linear falls back
    to for such shapes (:190-197)."""
    assert input_scale is None
    input_2d = input.view(-1, input.shape[-1])
    output_shape = [*input.shape[:-1], weight.shape[0]]
    q_input, x_scale = sglang_per_token_group_quant_fp8(input_2d, block_size[1], column_major_scales=False)
    output = w8a8_block_fp8_matmul(q_input, weight, x_scale, weight_scale, block_size, output_dtype=input_2d.dtype)
    if bias is not None:
        output += bias
    return output.to(dtype=input_2d.dtype).view(*output_shape)


# the name the reference's callers import for this branch
triton_w8a8_block_fp8_linear = ragged_w8a8_block_fp8_linear


def w8a8_block_fp8_linear(input: torch.Tensor, weight: torch.Tensor, block_size: List[int],
                          weight_scale: torch.Tensor, input_scale: Optional[torch.Tensor] = None,
                          bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`out` (extension): a row-major [tokens, N] tensor of the input dtype to write into."""
    assert input_scale is None
    assert list(block_size) == [128, 128]
    if weight.shape[0] % 128 != 0 or weight.shape[1] % 128 != 0:
        y = ragged_w8a8_block_fp8_linear(input, weight, block_size, weight_scale, input_scale, bias)
        if out is not None:
            out.copy_(y.view(out.shape))
            return out.view(y.shape)
        return y
    input_2d = input.view(-1, input.shape[-1])
    output_shape = [*input.shape[:-1], weight.shape[0]]
    q_input, x_scale = sglang_per_token_group_quant_fp8(
        input_2d, block_size[1], column_major_scales=True)
    output = fp8_blockwise_scaled_mm(q_input, weight.T, x_scale, weight_scale.T, out_dtype=input_2d.dtype, out=out)
    if bias is not None:
        output += bias
    return output.to(dtype=input_2d.dtype).view(*output_shape)


cutlass_w8a8_block_fp8_linear_with_fallback = w8a8_block_fp8_linear


def deepgemm_w8a8_block_fp8_linear_with_fallback(input: torch.Tensor, weight: torch.Tensor, block_size: List[int],
                                                 weight_scale: torch.Tensor,
                                                 input_scale: Optional[torch.Tensor] = None,
                                                 bias: Optional[torch.Tensor] = None,
                                                 scale_ue8m0: bool = True) -> torch.Tensor:
    """The reference's DeepGEMM linear (python/sglang/srt/layers/quantization/fp8_utils.py:215-258):
    activations quantised with column-major, 4-row-aligned scales -- power-of-two, packed UE8M0 when
    `scale_ue8m0` (the reference reads that switch from DEEPGEMM_SCALE_UE8M0, on for Blackwell) -- then the
    block-scaled product, bias, view back.  Shapes or dtypes the DeepGEMM path does not take fall back to
    the fp32-scale linear, as the reference falls back to its Triton kernel."""
    assert input_scale is None
    if not (input.dtype == torch.bfloat16 and weight.shape[0] % 64 == 0 and weight.shape[1] % 128 == 0
            and weight.shape[0] % 128 == 0):
        return w8a8_block_fp8_linear(input, weight, block_size, weight_scale, input_scale, bias)
    input_2d = input.view(-1, input.shape[-1])
    output_shape = [*input.shape[:-1], weight.shape[0]]
    q_input, x_scale = sglang_per_token_group_quant_fp8(input_2d, block_size[1], column_major_scales=True,
                                                        scale_tma_aligned=True, scale_ue8m0=scale_ue8m0)
    output = w8a8_block_fp8_matmul_deepgemm(q_input, weight, x_scale, weight_scale, block_size,
                                            output_dtype=input.dtype)
    if bias is not None:
        output += bias
    return output.to(dtype=input.dtype).view(*output_shape)


def dispatch_w8a8_block_fp8_linear() -> Callable:
    return w8a8_block_fp8_linear

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
from .fp8_kernel import sglang_per_token_group_quant_fp8


def w8a8_block_fp8_linear(input: torch.Tensor, weight: torch.Tensor, block_size: List[int],
                          weight_scale: torch.Tensor, input_scale: Optional[torch.Tensor] = None,
                          bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`out` (extension): a row-major [tokens, N] tensor of the input dtype to write into."""
    assert input_scale is None
    assert list(block_size) == [128, 128]
    input_2d = input.view(-1, input.shape[-1])
    output_shape = [*input.shape[:-1], weight.shape[0]]
    q_input, x_scale = sglang_per_token_group_quant_fp8(
        input_2d, block_size[1], column_major_scales=True)
    output = fp8_blockwise_scaled_mm(q_input, weight.T, x_scale, weight_scale.T, out_dtype=input_2d.dtype, out=out)
    if bias is not None:
        output += bias
    return output.to(dtype=input_2d.dtype).view(*output_shape)


cutlass_w8a8_block_fp8_linear_with_fallback = w8a8_block_fp8_linear


def dispatch_w8a8_block_fp8_linear() -> Callable:
    return w8a8_block_fp8_linear

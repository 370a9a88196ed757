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


def ceil_to_ue8m0(x: torch.Tensor) -> torch.Tensor:
    """2 ** ceil(log2(|x|)) (fp8_utils.py:485-486)."""
    return torch.pow(2.0, torch.ceil(torch.log2(x.abs())))


def requant_weight_ue8m0(weight: torch.Tensor, weight_scale_inv: torch.Tensor, weight_block_size: List[int]):
    """Block-quantised weight [..., N, K] (e4m3) + fp32 block scales -> the same weight re-quantised with
    POWER-OF-TWO block scales: dequantise to bf16, block amax (floor 1e-4), scale = 2 ** ceil(log2(amax / 448)),
    codes = e4m3(w / scale).  The arithmetic of the reference's _requant_weight_ue8m0 / per_block_cast_to_fp8
    (python/sglang/srt/layers/quantization/fp8_utils.py:421-481); the scales stay fp32 [..., N/128, K/128] here
    (the reference repacks them for DeepGEMM), which is what b200_fp8_blockwise_scaled_mm_pow2 takes."""
    assert list(weight_block_size) == [128, 128]
    *lead, n, k = weight.shape
    s_rep = weight_scale_inv.repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)[..., :n, :k]
    w = (weight.to(torch.float32) * s_rep).to(torch.bfloat16).reshape(-1, k)
    rows = w.shape[0]
    assert n % 128 == 0 or not lead, "stacked weights need N % 128 == 0"
    pr, pk = (rows + 127) // 128 * 128, (k + 127) // 128 * 128
    wp = torch.zeros((pr, pk), dtype=w.dtype, device=w.device)
    wp[:rows, :k] = w
    wv = wp.view(-1, 128, pk // 128, 128)
    amax = wv.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    sf = ceil_to_ue8m0(amax / 448.0)
    q = (wv * (1.0 / sf)).to(torch.float8_e4m3fn).view(pr, pk)[:rows, :k].contiguous()
    return q.view(weight.shape), sf.view(pr // 128, pk // 128).view(weight_scale_inv.shape).contiguous()


def requant_weight_ue8m0_inplace(weight, weight_scale_inv, weight_block_size) -> None:
    """fp8_utils.py:413-418."""
    assert isinstance(weight, torch.nn.Parameter) and isinstance(weight_scale_inv, torch.nn.Parameter)
    weight.data, weight_scale_inv.data = requant_weight_ue8m0(weight.data, weight_scale_inv.data, weight_block_size)


def deepgemm_w8a8_block_fp8_linear_with_fallback(input: torch.Tensor, weight: torch.Tensor, block_size: List[int],
                                                 weight_scale: torch.Tensor,
                                                 input_scale: Optional[torch.Tensor] = None,
                                                 bias: Optional[torch.Tensor] = None,
                                                 scale_ue8m0: bool = True,
                                                 weight_scale_ue8m0: bool = False) -> torch.Tensor:
    """The reference's DeepGEMM linear (python/sglang/srt/layers/quantization/fp8_utils.py:215-258):
    activations quantised with column-major, 4-row-aligned scales -- power-of-two, packed UE8M0 when
    `scale_ue8m0` (the reference reads that switch from DEEPGEMM_SCALE_UE8M0, on for Blackwell) -- then the
    block-scaled product, bias, view back.  Shapes or dtypes the DeepGEMM path does not take fall back to
    the fp32-scale linear, as the reference falls back to its Triton kernel.  weight_scale_ue8m0=True promises
    power-of-two weight scales too (requant_weight_ue8m0): the product then runs on the tensor core's
    block-scaling path, all k-blocks accumulated in tensor memory."""
    assert input_scale is None
    if not (input.dtype == torch.bfloat16 and weight.shape[0] % 64 == 0 and weight.shape[1] % 128 == 0
            and weight.shape[0] % 128 == 0):
        return w8a8_block_fp8_linear(input, weight, block_size, weight_scale, input_scale, bias)
    input_2d = input.view(-1, input.shape[-1])
    output_shape = [*input.shape[:-1], weight.shape[0]]
    q_input, x_scale = sglang_per_token_group_quant_fp8(input_2d, block_size[1], column_major_scales=True,
                                                        scale_tma_aligned=True, scale_ue8m0=scale_ue8m0)
    output = w8a8_block_fp8_matmul_deepgemm(q_input, weight, x_scale, weight_scale, block_size,
                                            output_dtype=input.dtype,
                                            weight_scale_ue8m0=bool(weight_scale_ue8m0 and scale_ue8m0))
    if bias is not None:
        output += bias
    return output.to(dtype=input.dtype).view(*output_shape)


def dispatch_w8a8_block_fp8_linear() -> Callable:
    return w8a8_block_fp8_linear

"""Per-token-group INT8 quantisation: the int8 destination of the operator the block-FP8 path quantises with.

Mirrors `sglang_per_token_group_quant_int8` (python/sglang/srt/layers/quantization/int8_kernel.py:185-209): same
name, arguments, return value and assertions, backed by `sgl_kernel.sgl_per_token_group_quant_int8`
(sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:219-228).  Only the quantiser is built; the INT8 matmul of
that file is a different path.
"""
from __future__ import annotations

from typing import Tuple

import torch

from ...sgl_kernel import sgl_per_token_group_quant_int8


def sglang_per_token_group_quant_int8(x: torch.Tensor, group_size: int, eps: float = 1e-10,
                                      dtype: torch.dtype = torch.int8) -> Tuple[torch.Tensor, torch.Tensor]:
    assert x.shape[-1] % group_size == 0, "the last dimension of `x` cannot be divisible by `group_size`"
    assert x.is_contiguous(), "`x` is not contiguous"
    iinfo = torch.iinfo(dtype)
    x_q = torch.empty_like(x, device=x.device, dtype=dtype)
    x_s = torch.empty(x.shape[:-1] + (x.shape[-1] // group_size,), device=x.device, dtype=torch.float32)
    if x.numel() > 0:
        sgl_per_token_group_quant_int8(x, x_q, x_s.view(-1, x_s.shape[-1]), group_size, eps, iinfo.min, iinfo.max)
    return x_q, x_s

"""sglang-level functions of the block-FP8 path, same names and signatures as
python/sglang/srt/layers/quantization/fp8_kernel.py in the reference:

  create_per_token_group_quant_fp8_output_scale   :300-341
  sglang_per_token_group_quant_fp8                :344-372
  per_token_group_quant_fp8                       :209-297 (the Triton twin; same results here)
  w8a8_block_fp8_matmul                           :849-966 (prepare_block_fp8_matmul_inputs :801-846)
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ...sgl_kernel import fp8_blockwise_scaled_mm, sgl_per_token_group_quant_fp8
from ...sgl_kernel.gemm import launch_dense_mm
from ... import _lib

fp8_dtype = torch.float8_e4m3fn
fp8_max = torch.finfo(fp8_dtype).max
fp8_min = -fp8_max


def create_per_token_group_quant_fp8_output_scale(x_shape, device, group_size, column_major_scales: bool,
                                                  scale_tma_aligned: bool, scale_ue8m0: bool):
    if scale_ue8m0:
        # biased-exponent bytes, four k-groups per int32, column-major and padded to 4 rows / 4 groups
        # (python/sglang/srt/layers/quantization/fp8_kernel.py:308-319); zero-filled like the reference
        assert column_major_scales and scale_tma_aligned
        assert group_size == 128 and len(x_shape) == 2
        x_q_mn, x_q_k = x_shape
        aligned_mn = (x_q_mn + 3) // 4 * 4
        aligned_k = (x_q_k // 128 + 3) // 4 * 4
        return torch.zeros((aligned_k // 4, aligned_mn), device=device, dtype=torch.int).transpose(0, 1)[:x_q_mn, :]
    if column_major_scales:
        if scale_tma_aligned:
            aligned_size = (x_shape[-2] + 3) // 4 * 4
            return torch.empty(x_shape[:-2] + (x_shape[-1] // group_size, aligned_size), device=device,
                               dtype=torch.float32).permute(-1, -2)[: x_shape[-2], :]
        return torch.empty((x_shape[-1] // group_size,) + x_shape[:-1], device=device,
                           dtype=torch.float32).permute(-1, -2)
    return torch.empty(x_shape[:-1] + (x_shape[-1] // group_size,), device=device, dtype=torch.float32)


def sglang_per_token_group_quant_fp8(x: torch.Tensor, group_size: int, eps: float = 1e-10,
                                     column_major_scales: bool = False, scale_tma_aligned: bool = False,
                                     scale_ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    assert x.shape[-1] % group_size == 0, "the last dimension of `x` cannot be divisible by `group_size`"
    assert x.is_contiguous(), "`x` is not contiguous"
    x_q = torch.empty_like(x, device=x.device, dtype=fp8_dtype)
    x_s = create_per_token_group_quant_fp8_output_scale(
        x_shape=x.shape, device=x.device, group_size=group_size, column_major_scales=column_major_scales,
        scale_tma_aligned=scale_tma_aligned, scale_ue8m0=scale_ue8m0)
    if x.shape[0] > 0:
        sgl_per_token_group_quant_fp8(x, x_q, x_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0)
    return x_q, x_s


def per_token_group_quant_fp8_ue8m0_rows(x: torch.Tensor, eps: float = 1e-10) -> Tuple[torch.Tensor, torch.Tensor]:
    """The power-of-two quantisation (same codes and exponent bytes as sglang_per_token_group_quant_fp8 with
    scale_ue8m0=True) with every token's packed words CONTIGUOUS: scales int32 [M, W], W = ceil(K / 512) rounded up to
    four words (16 bytes), padding words zero.  One scale row per token is what the expert-parallel dispatch copies;
    the grouped block-scaling GEMM takes the layout through its strides."""
    assert x.dim() == 2 and x.is_contiguous() and x.shape[1] % 128 == 0
    M, K = x.shape
    W = ((K // 128 + 3) // 4 + 3) // 4 * 4
    x_q = torch.empty_like(x, dtype=fp8_dtype)
    x_s = torch.zeros((M, W), dtype=torch.int32, device=x.device)
    if M > 0:
        dt = {torch.float32: _lib.DT_F32, torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16}[x.dtype]
        with torch.cuda.device(x.device):
            rc = _lib.lib().b200_per_token_group_quant_fp8_ue8m0_strided(
                x.data_ptr(), dt, x_q.data_ptr(), x_s.data_ptr(), M, K, W, 1, eps, fp8_min, fp8_max,
                torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check("per_token_group_quant_fp8_ue8m0_rows", rc)
    return x_q, x_s


def silu_and_mul_per_token_group_quant_fp8(x: torch.Tensor, group_size: int = 128, eps: float = 1e-10,
                                           column_major_scales: bool = False, scale_tma_aligned: bool = False,
                                           scale_ue8m0: bool = False):
    """x [..., 2K] (gate | up) -> codes [..., K], scales as in sglang_per_token_group_quant_fp8.
    Bit-identical to silu_and_mul followed by sglang_per_token_group_quant_fp8; one kernel, and the
    [..., K] intermediate is never written.  (The reference has this fusion only as a Triton kernel
    in its EP path: python/sglang/srt/layers/moe/ep_moe/kernels.py:317-460.)"""
    assert group_size == 128, "the fused form is built for 128-wide groups"
    assert x.is_contiguous() and x.shape[-1] % 256 == 0
    assert x.dtype in (torch.bfloat16, torch.float16)
    K = x.shape[-1] // 2
    out_shape = x.shape[:-1] + (K,)
    M = x.numel() // (2 * K)
    x_q = torch.empty(out_shape, device=x.device, dtype=fp8_dtype)
    dt = {torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16}[x.dtype]
    if scale_ue8m0:
        x_s = create_per_token_group_quant_fp8_output_scale((M, K), x.device, group_size, True, True, True)
        if M > 0:
            with torch.cuda.device(x.device):
                rc = _lib.lib().b200_silu_mul_per_token_group_quant_fp8_ue8m0(
                    x.data_ptr(), dt, x_q.data_ptr(), x_s.data_ptr(), M, K, x_s.stride(1), eps, fp8_min, fp8_max,
                    torch.cuda.current_stream(x.device).cuda_stream)
            _lib.check("silu_and_mul_per_token_group_quant_fp8", rc)
        return x_q, x_s
    x_s = create_per_token_group_quant_fp8_output_scale(out_shape, x.device, group_size, column_major_scales,
                                                        scale_tma_aligned, False)
    if M > 0:
        s2 = x_s.reshape(M, K // 128) if x_s.dim() != 2 else x_s
        with torch.cuda.device(x.device):
            rc = _lib.lib().b200_silu_mul_per_token_group_quant_fp8(
                x.data_ptr(), dt, x_q.data_ptr(), s2.data_ptr(), M, K, s2.stride(0), s2.stride(1), eps, fp8_min,
                fp8_max, torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check("silu_and_mul_per_token_group_quant_fp8", rc)
    return x_q, x_s


def gather_per_token_group_quant_fp8(x: torch.Tensor, src_rows: torch.Tensor, group_size: int = 128, eps: float = 1e-10,
                                     column_major_scales: bool = False, scale_tma_aligned: bool = False,
                                     scale_ue8m0: bool = False):
    """Row r of the result = codes and scales of x[src_rows[r]]: sglang_per_token_group_quant_fp8 followed by a row
    gather of codes and scales (shuffle_rows in the reference's cutlass_moe.py:144-150; ep_scatter in its EP path),
    in one kernel and with the same bits.  x [M, K] bf16/fp16/fp32 contiguous, src_rows [R] int32."""
    assert group_size == 128, "the fused form is built for 128-wide groups"
    assert x.dim() == 2 and x.is_contiguous() and x.shape[1] % 128 == 0
    assert src_rows.dtype == torch.int32 and src_rows.is_contiguous()
    M, K = x.shape
    R = src_rows.numel()
    x_q = torch.empty((R, K), device=x.device, dtype=fp8_dtype)
    x_s = create_per_token_group_quant_fp8_output_scale((R, K), x.device, group_size, column_major_scales,
                                                        scale_tma_aligned, scale_ue8m0)
    if R > 0:
        dt = {torch.float32: _lib.DT_F32, torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16}[x.dtype]
        with torch.cuda.device(x.device):
            rc = _lib.lib().b200_gather_per_token_group_quant_fp8(
                x.data_ptr(), dt, M, src_rows.data_ptr(), x_q.data_ptr(), x_s.data_ptr(), R, K, x_s.stride(0),
                x_s.stride(1), 1 if scale_ue8m0 else 0, eps, fp8_min, fp8_max,
                torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check("gather_per_token_group_quant_fp8", rc)
    return x_q, x_s


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None):
    """RMSNorm.forward_native's arithmetic (python/sglang/srt/layers/layernorm.py:135-171) in one kernel: returns the
    normalised tensor; with `residual`, x + residual is normalised and `residual` is overwritten with the sum."""
    _, y, _, _ = _rmsnorm_launch(x, weight, eps, residual, want_y=True, want_q=False)
    return y


def rmsnorm_per_token_group_quant_fp8(x: torch.Tensor, weight: torch.Tensor, norm_eps: float = 1e-6,
                                      residual: Optional[torch.Tensor] = None, group_size: int = 128,
                                      eps: float = 1e-10, column_major_scales: bool = False,
                                      scale_tma_aligned: bool = False, scale_ue8m0: bool = False,
                                      return_normed: bool = False):
    """RMSNorm (optionally with the residual add) and the group quantisation of its output in one pass: bit-identical
    to rmsnorm(...) followed by sglang_per_token_group_quant_fp8(...), without writing and re-reading the normalised
    activations.  Returns (codes, scales) or (codes, scales, normed) with return_normed."""
    assert group_size == 128, "the fused form is built for 128-wide groups"
    _, y, q, s = _rmsnorm_launch(x, weight, norm_eps, residual, want_y=return_normed, want_q=True, eps=eps,
                                 column_major_scales=column_major_scales, scale_tma_aligned=scale_tma_aligned,
                                 scale_ue8m0=scale_ue8m0)
    return (q, s, y) if return_normed else (q, s)


def _rmsnorm_launch(x, weight, norm_eps, residual, want_y, want_q, eps=1e-10, column_major_scales=False,
                    scale_tma_aligned=False, scale_ue8m0=False):
    assert x.is_contiguous() and x.dtype in (torch.bfloat16, torch.float16)
    K = x.shape[-1]
    assert weight.shape == (K,) and weight.dtype == x.dtype and weight.is_contiguous()
    assert K % 128 == 0 and K <= 16384
    if residual is not None:
        assert residual.shape == x.shape and residual.dtype == x.dtype and residual.is_contiguous()
    M = x.numel() // K
    y = torch.empty_like(x) if want_y else None
    q = s = None
    ssr = ssg = 0
    if want_q:
        q = torch.empty(x.shape, device=x.device, dtype=fp8_dtype)
        s = create_per_token_group_quant_fp8_output_scale((M, K) if scale_ue8m0 else x.shape, x.device, 128,
                                                          column_major_scales, scale_tma_aligned, scale_ue8m0)
        s2 = s if s.dim() == 2 else s.reshape(M, K // 128)
        ssr, ssg = s2.stride(0), s2.stride(1)
    if M > 0:
        dt = {torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16}[x.dtype]
        with torch.cuda.device(x.device):
            rc = _lib.lib().b200_rmsnorm_per_token_group_quant_fp8(
                x.data_ptr(), dt, residual.data_ptr() if residual is not None else None, weight.data_ptr(),
                float(norm_eps), y.data_ptr() if y is not None else None, q.data_ptr() if q is not None else None,
                s.data_ptr() if s is not None else None, M, K, ssr, ssg, 1 if scale_ue8m0 else 0, eps, fp8_min, fp8_max,
                torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check("rmsnorm_per_token_group_quant_fp8", rc)
    return residual, y, q, s


def per_token_group_quant_fp8(x: torch.Tensor, group_size: int, eps: float = 1e-10,
                              column_major_scales: bool = False, scale_tma_aligned: bool = False,
                              scale_ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same contract as the reference's Triton entry; one kernel serves both names here."""
    return sglang_per_token_group_quant_fp8(x, group_size, eps, column_major_scales, scale_tma_aligned, scale_ue8m0)


def w8a8_block_fp8_matmul(A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor,
                          block_size: List[int], output_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """A [...,K] e4m3 contiguous; B [N,K] e4m3 contiguous; As [...,ceil(K/128)] fp32 (any strides);
    Bs [ceil(N/128), ceil(K/128)] fp32; returns [...,N] in output_dtype."""
    assert len(block_size) == 2
    block_n, block_k = block_size
    assert block_n == 128 and block_k == 128, "only 128x128 weight blocks are built"
    assert A.shape[-1] == B.shape[-1]
    assert A.shape[:-1] == As.shape[:-1]
    assert A.is_contiguous()
    assert (A.shape[-1] + block_k - 1) // block_k == As.shape[-1]
    M = A.numel() // A.shape[-1]
    assert B.ndim == 2 and B.is_contiguous() and Bs.ndim == 2
    N, K = B.shape
    assert (N + block_n - 1) // block_n == Bs.shape[0]
    assert (K + block_k - 1) // block_k == Bs.shape[1]
    assert A.dtype == fp8_dtype and B.dtype == fp8_dtype
    C = A.new_empty(A.shape[:-1] + (N,), dtype=output_dtype)
    if M == 0:
        return C
    As2 = As.reshape(M, As.shape[-1]) if As.dim() != 2 else As
    dt = {torch.float32: _lib.DT_F32, torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16}[output_dtype]
    rc = launch_dense_mm((A.data_ptr(), K, B.data_ptr(), K, As2.data_ptr(), As2.stride(0), As2.stride(1),
                          Bs.data_ptr(), Bs.stride(0), Bs.stride(1), C.data_ptr(), N, dt, M, N, K), M, N, K, A.device)
    _lib.check("w8a8_block_fp8_matmul", rc)
    return C


def w8a8_block_fp8_matmul_deepgemm(A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor,
                                   block_size: List[int], output_dtype: torch.dtype,
                                   weight_scale_ue8m0: bool = False) -> torch.Tensor:
    """C = A @ B.T with block scales where `As` may be the packed UE8M0 tensor that
    sglang_per_token_group_quant_fp8(..., scale_ue8m0=True) returns (int32 [M, ceil(K/512)], rows contiguous)
    or fp32 scales [M, K/128]; `Bs` fp32 [N/128, K/128].  Mirrors the call surface of the reference's
    w8a8_block_fp8_matmul_deepgemm (python/sglang/srt/layers/quantization/fp8_kernel.py:849-867); bf16 only,
    like DeepGEMM.  weight_scale_ue8m0=True promises that `Bs` holds powers of two as well (what the reference's
    requant_weight_ue8m0 leaves, fp8_utils.py:370-443): the product then runs on the tensor core's block-scaling
    path with every k-block accumulated in tensor memory."""
    assert list(block_size) == [128, 128] and output_dtype == torch.bfloat16
    if As.dtype != torch.int32:
        return w8a8_block_fp8_matmul(A, B, As, Bs, block_size, output_dtype)
    assert A.dim() == 2 and A.is_contiguous() and B.dim() == 2 and B.is_contiguous()
    M, K = A.shape
    N = B.shape[0]
    assert B.shape[1] == K and K % 128 == 0 and N % 128 == 0
    assert A.dtype == fp8_dtype and B.dtype == fp8_dtype and Bs.dtype == torch.float32
    assert As.shape == (M, (K // 128 + 3) // 4) and (As.stride(0) == 1 or M == 1), "packed scales must be column-major"
    assert Bs.shape == (N // 128, K // 128)
    C = torch.empty((M, N), dtype=output_dtype, device=A.device)
    if M == 0:
        return C
    with torch.cuda.device(A.device):
        entry = _lib.lib().b200_fp8_blockwise_scaled_mm_pow2 if weight_scale_ue8m0 else \
            _lib.lib().b200_fp8_blockwise_scaled_mm_ue8m0
        rc = entry(
            A.data_ptr(), K, B.data_ptr(), K, As.data_ptr(), As.stride(0), As.stride(1),
            Bs.data_ptr(), Bs.stride(0), Bs.stride(1), C.data_ptr(), N, _lib.DT_BF16, M, N, K,
            torch.cuda.current_stream(A.device).cuda_stream)
    _lib.check("w8a8_block_fp8_matmul_deepgemm", rc)
    return C

"""The DeepGEMM call surface of the reference on Blackwell, served by this library's block-scaling kernel
(gemm_mx.cu: tcgen05.mma kind::mxf8f6f4.block_scale, every k-block accumulated in tensor memory).

Same names and argument order as python/sglang/srt/layers/quantization/deep_gemm_wrapper/entrypoint.py:

  gemm_nt_f8f8bf16                  :78-93    (deep_gemm.fp8_gemm_nt)
  grouped_gemm_nt_f8f8bf16_contig   :62-75    (deep_gemm.m_grouped_fp8_gemm_nt_contiguous)
  grouped_gemm_nt_f8f8bf16_masked   :39-59    (deep_gemm.fp8_m_grouped_gemm_nt_masked)

lhs = (codes, scales): e4m3 codes and the PACKED power-of-two activation scales that
sglang_per_token_group_quant_fp8(..., column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
writes -- int32, four k-groups per word, rows contiguous.  rhs = (weights, scales): e4m3 [.., N, K] and fp32
block scales [.., N/128, K/128] that hold powers of two (requant_weight_ue8m0; the reference repacks them into
DeepGEMM's integer layout, this library reads the exponent field of the fp32 value instead).  bf16 output, like
DeepGEMM.  Both grouped layouts are special cases of one device-resident problem table
(b200_fp8_blockwise_scaled_grouped_mm_pow2); nothing here reads a count on the host.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ... import _lib

DEEPGEMM_BLACKWELL = True
DEEPGEMM_SCALE_UE8M0 = True
M_ALIGNMENT_CONTIGUOUS = 128     # deep_gemm.get_m_alignment_for_contiguous_layout()

fp8_dtype = torch.float8_e4m3fn


def get_m_alignment_for_contiguous_layout() -> int:
    return M_ALIGNMENT_CONTIGUOUS


def grouped_gemm_pow2(a: torch.Tensor, sa_packed: torch.Tensor, w: torch.Tensor, ws: torch.Tensor, out: torch.Tensor,
                      problem_offsets: torch.Tensor, problem_rows: torch.Tensor,
                      problem_experts: Optional[torch.Tensor] = None, sa_stride_problem: int = -1) -> torch.Tensor:
    """The general form.  a [R, K] e4m3 and out [R, N] row-major; w [E, N, K] e4m3 contiguous; ws [E, N/128, K/128]
    fp32 powers of two (any strides).  Problem i multiplies rows [problem_offsets[i], + problem_rows[i]) with expert
    problem_experts[i] (i when None; a negative id skips the problem).  problem_rows may be a strided int32 view
    (column 0 of the reference's problem_sizes).  sa_packed: packed exponents, word (row, g4) at
    `g4 * stride(1) + row * stride(0)` for the global row (sa_stride_problem < 0), else per problem with the row
    counted inside the problem and the problem's words starting `sa_stride_problem` words apart."""
    R, K = a.shape
    E, N, Kw = w.shape
    assert Kw == K and K % 128 == 0 and N % 128 == 0
    assert a.dtype == fp8_dtype and w.dtype == fp8_dtype and a.is_contiguous() and w.is_contiguous()
    assert sa_packed.dtype == torch.int32 and ws.dtype == torch.float32 and ws.shape == (E, N // 128, K // 128)
    assert sa_packed.shape[-1] >= (K // 128 + 3) // 4, "one packed word per four k-blocks"
    assert out.shape == (R, N) and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float16, torch.float32)
    assert problem_offsets.dtype == torch.int32 and problem_rows.dtype == torch.int32
    assert problem_offsets.is_contiguous() and problem_rows.dim() == 1
    P = problem_offsets.numel()
    assert problem_rows.numel() == P
    if problem_experts is not None:
        assert problem_experts.dtype == torch.int32 and problem_experts.is_contiguous() and problem_experts.numel() == P
    if R == 0 or P == 0:
        return out
    dt = {torch.float32: _lib.DT_F32, torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16}[out.dtype]
    with torch.cuda.device(a.device):
        rc = _lib.lib().b200_fp8_blockwise_scaled_grouped_mm_pow2(
            a.data_ptr(), K, R, w.data_ptr(), K, sa_packed.data_ptr(), sa_packed.stride(-2), sa_packed.stride(-1),
            sa_stride_problem, ws.data_ptr(), ws.stride(0), ws.stride(1), ws.stride(2), out.data_ptr(), out.stride(0),
            dt, problem_offsets.data_ptr(), problem_rows.data_ptr(), problem_rows.stride(0),
            problem_experts.data_ptr() if problem_experts is not None else None, P, E, N, K,
            torch.cuda.current_stream(a.device).cuda_stream)
    _lib.check("grouped_gemm_pow2", rc)
    return out


def grouped_gemm_pow2_silu_quant(a: torch.Tensor, sa_packed: torch.Tensor, w13: torch.Tensor, w13s: torch.Tensor,
                                 problem_offsets: torch.Tensor, problem_rows: torch.Tensor,
                                 problem_experts: Optional[torch.Tensor] = None, mid_dtype: torch.dtype = torch.bfloat16,
                                 sa_stride_problem: int = -1):
    """Expert GEMM 1 with SiLU*mul and the next GEMM's power-of-two quantisation in its epilogue.  a [R, K] e4m3,
    w13 [E, 2n, K] (gate rows first), w13s [E, 2n/128, K/128] fp32 powers of two.  Returns (codes [R, n] e4m3, packed
    exponents int32 [R, ceil(n/512)], rows contiguous) -- the bits of grouped_gemm_pow2 into a `mid_dtype` tensor
    followed by silu_and_mul_per_token_group_quant_fp8(..., scale_ue8m0=True)."""
    from .fp8_kernel import create_per_token_group_quant_fp8_output_scale
    R, K = a.shape
    E, n2, Kw = w13.shape
    n = n2 // 2
    assert Kw == K and K % 128 == 0 and n % 128 == 0 and n2 == 2 * n
    assert a.dtype == fp8_dtype and w13.dtype == fp8_dtype and a.is_contiguous() and w13.is_contiguous()
    assert sa_packed.dtype == torch.int32 and w13s.dtype == torch.float32 and w13s.shape == (E, n2 // 128, K // 128)
    assert problem_offsets.dtype == torch.int32 and problem_rows.dtype == torch.int32 and problem_rows.dim() == 1
    P = problem_offsets.numel()
    q = torch.empty((R, n), dtype=fp8_dtype, device=a.device)
    s = create_per_token_group_quant_fp8_output_scale((R, n), a.device, 128, True, True, True)     # zero-filled
    if R == 0 or P == 0:
        return q, s
    dt = {torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16}[mid_dtype]
    with torch.cuda.device(a.device):
        rc = _lib.lib().b200_fp8_blockwise_scaled_grouped_mm_pow2_silu_quant(
            a.data_ptr(), K, R, w13.data_ptr(), K, sa_packed.data_ptr(), sa_packed.stride(-2), sa_packed.stride(-1),
            sa_stride_problem, w13s.data_ptr(), w13s.stride(0), w13s.stride(1), w13s.stride(2), q.data_ptr(), n,
            s.data_ptr(), s.stride(1), dt, problem_offsets.data_ptr(), problem_rows.data_ptr(), problem_rows.stride(0),
            problem_experts.data_ptr() if problem_experts is not None else None, P, E, n, K,
            torch.cuda.current_stream(a.device).cuda_stream)
    _lib.check("grouped_gemm_pow2_silu_quant", rc)
    return q, s


def gate_up_silu_quant_pow2(a: torch.Tensor, sa_packed: torch.Tensor, w_gate_up: torch.Tensor, ws: torch.Tensor,
                            mid_dtype: torch.dtype = torch.bfloat16):
    """Dense MLP, first half, on the block-scaling path: a [M, K] e4m3 with packed exponents, w_gate_up [2n, K]
    (gate rows first: the merged gate_up weight of the reference's MergedColumnParallelLinear,
    python/sglang/srt/layers/linear.py:415-520), ws [2n/128, K/128] fp32 powers of two.  One kernel computes the
    projection, SiLU(gate) * up and the quantisation for the down projection; returns (codes [M, n], packed exponents).
    Same bits as the GEMM into a `mid_dtype` tensor followed by silu_and_mul_per_token_group_quant_fp8."""
    M = a.shape[0]
    dev = a.device
    offsets = torch.zeros(1, dtype=torch.int32, device=dev)
    rows = torch.full((1,), M, dtype=torch.int32, device=dev)
    return grouped_gemm_pow2_silu_quant(a, sa_packed, w_gate_up.unsqueeze(0), ws.unsqueeze(0), offsets, rows,
                                        mid_dtype=mid_dtype)


def gemm_nt_f8f8bf16(lhs: Tuple[torch.Tensor, torch.Tensor], rhs: Tuple[torch.Tensor, torch.Tensor],
                     out: torch.Tensor) -> None:
    """out[M, N] = lhs[M, K] @ rhs[N, K].T (entrypoint.py:78-93)."""
    a, sa = lhs
    b, sb = rhs
    assert out.dtype == torch.bfloat16 and out.is_contiguous()
    m, k = a.shape
    n = b.shape[0]
    assert out.shape == (m, n) and k % 128 == 0 and n % 128 == 0 and b.shape[1] == k
    assert a.dtype == fp8_dtype and b.dtype == fp8_dtype and a.is_contiguous() and b.is_contiguous()
    assert sa.dtype == torch.int32 and sb.dtype == torch.float32 and sb.shape == (n // 128, k // 128)
    if m == 0:
        return
    with torch.cuda.device(a.device):
        rc = _lib.lib().b200_fp8_blockwise_scaled_mm_pow2(
            a.data_ptr(), k, b.data_ptr(), k, sa.data_ptr(), sa.stride(0), sa.stride(1), sb.data_ptr(), sb.stride(0),
            sb.stride(1), out.data_ptr(), n, _lib.DT_BF16, m, n, k, torch.cuda.current_stream(a.device).cuda_stream)
    _lib.check("gemm_nt_f8f8bf16", rc)


def grouped_gemm_nt_f8f8bf16_contig(lhs: Tuple[torch.Tensor, torch.Tensor], rhs: Tuple[torch.Tensor, torch.Tensor],
                                    out: torch.Tensor, m_indices: torch.Tensor) -> None:
    """Contiguous layout (entrypoint.py:62-75; caller python/sglang/srt/layers/moe/ep_moe/layer.py:540-640): the
    rows of all experts in one [M, K] tensor, every expert's run padded to a multiple of 128 rows, m_indices[r] =
    expert of row r (negative = padding that belongs to nobody).  Each 128-row block is one problem whose expert
    is read from m_indices on the device."""
    a, sa = lhs
    w, ws = rhs
    M, K = a.shape
    assert M % M_ALIGNMENT_CONTIGUOUS == 0, "the contiguous layout pads every expert's rows to 128"
    assert m_indices.dtype == torch.int32 and m_indices.numel() == M
    blocks = M // M_ALIGNMENT_CONTIGUOUS
    if blocks == 0:
        return
    experts = m_indices[::M_ALIGNMENT_CONTIGUOUS].contiguous()
    offsets = torch.arange(0, M, M_ALIGNMENT_CONTIGUOUS, dtype=torch.int32, device=a.device)
    rows = torch.full((blocks,), M_ALIGNMENT_CONTIGUOUS, dtype=torch.int32, device=a.device)
    grouped_gemm_pow2(a, sa, w, ws, out, offsets, rows, experts)


def grouped_gemm_nt_f8f8bf16_masked(lhs: Tuple[torch.Tensor, torch.Tensor], rhs: Tuple[torch.Tensor, torch.Tensor],
                                    out: torch.Tensor, masked_m: torch.Tensor, expected_m: int, recipe=None) -> None:
    """Masked layout (entrypoint.py:39-59; caller ep_moe/layer.py:205-320): lhs codes [E, max_m, K], of which the
    first masked_m[e] rows of expert e are valid; packed scales [E, max_m, K/512] int32 with the rows of an expert
    contiguous (what _cast_to_e8m0_with_rounding_up leaves, ep_moe/layer.py:62-72); out [E, max_m, N].  Rows past
    masked_m[e] are not computed and not written.  `expected_m` is a tuning hint of DeepGEMM; unused."""
    a, sa = lhs
    w, ws = rhs
    E, max_m, K = a.shape
    N = w.shape[1]
    assert out.shape == (E, max_m, N) and out.is_contiguous() and a.is_contiguous()
    assert masked_m.dtype == torch.int32 and masked_m.numel() == E and masked_m.is_contiguous()
    assert sa.dim() == 3 and sa.shape[0] == E and sa.shape[1] == max_m
    offsets = torch.arange(0, E * max_m, max_m, dtype=torch.int32, device=a.device)
    rows = torch.clamp(masked_m, max=max_m)
    grouped_gemm_pow2(a.view(E * max_m, K), sa, w, ws, out.view(E * max_m, N), offsets, rows, None,
                      sa_stride_problem=sa.stride(0))

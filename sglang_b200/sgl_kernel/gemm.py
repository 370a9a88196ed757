"""Python surface of the reference's `sgl_kernel.gemm` for the block-FP8 path, backed by the
B200 C-ABI library.

Mirrors (names, argument order, layouts, error behaviour):
  sgl_kernel.fp8_blockwise_scaled_mm          sgl-kernel/python/sgl_kernel/gemm.py:24-31
  sgl_kernel.sgl_per_token_group_quant_fp8    sgl-kernel/python/sgl_kernel/gemm.py:100-112
  sgl_kernel.sgl_per_token_group_quant_int8   sgl-kernel/python/sgl_kernel/gemm.py:115-126
and the argument checks of the C++ entry points they dispatch to
(sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:351-383,
 sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:125-131,153-156).
"""
from __future__ import annotations

import torch

from .. import _lib

FP8 = torch.float8_e4m3fn

_DT = {torch.float32: _lib.DT_F32, torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16}


def _check(cond: bool, msg: str) -> None:
    # TORCH_CHECK -> c10::Error -> RuntimeError on the Python side
    if not cond:
        raise RuntimeError(msg)


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _is_contiguous_vector(t: torch.Tensor) -> bool:
    return t.is_contiguous() and (t.dim() == 1 or (t.dim() == 2 and min(t.shape) == 1))


_SM_COUNT: dict = {}
_WORKSPACE: dict = {}
# Split-K for decode-size batches: "auto" lets the library choose, "off" always runs the unsplit kernel.
SPLIT_K_MODE = "auto"


_PLAN: dict = {}
_SM_LIMIT = 0


def set_sm_limit(sms: int) -> int:
    """At most `sms` SMs for the persistent kernels launched from now on (0 = all); returns the previous limit.
    The counterpart of the reference's configure_deep_gemm_num_sms (deep_gemm_wrapper/entrypoint.py:100-110)."""
    global _SM_LIMIT
    old = _lib.lib().b200_set_sm_limit(int(sms))
    _SM_LIMIT = max(0, int(sms))
    return old


def _splitk_plan(M: int, N: int, K: int, device: torch.device):
    """Split count and workspace bytes the library chooses for this shape (1, 0 = no split): all tiles
    for decode-size M on narrow deep projections, only the last wave of tiles for large M when that wave
    would be mostly empty.  Cached per shape and device."""
    if SPLIT_K_MODE != "auto":
        return 1, 0
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (M, N, K, idx, _SM_LIMIT)
    hit = _PLAN.get(key)
    if hit is not None:
        return hit
    sms = _SM_COUNT.get(idx)
    if sms is None:
        sms = _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    if _SM_LIMIT > 0:
        sms = min(sms, _SM_LIMIT)
    import ctypes
    s, b = ctypes.c_int(1), ctypes.c_size_t(0)
    _lib.check("fp8_blockwise_scaled_mm_splitk_plan",
               _lib.lib().b200_fp8_blockwise_scaled_mm_splitk_plan(M, N, K, sms, ctypes.byref(s), ctypes.byref(b)))
    _PLAN[key] = (s.value, b.value)
    return _PLAN[key]


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Per-(device, stream) split-K workspace, grown on demand and reused: kernels on one stream run in
    order, so consecutive calls may share it; a different stream gets its own."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _WORKSPACE.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = _WORKSPACE[key] = torch.empty(max(nbytes, 1 << 22), dtype=torch.uint8, device=device)
    return ws


def launch_dense_mm(args: tuple, M: int, N: int, K: int, device: torch.device) -> int:
    """Enqueue the dense block-scaled GEMM on the current stream of `device`; `args` are the C-ABI arguments up to
    and including K.  Asks the split plan (cached) and passes a per-stream workspace when the library wants one:
    k-blocks of tiles that would leave most SMs idle are spread over those SMs.  Returns the C-ABI status."""
    with torch.cuda.device(device):
        split_k, ws_bytes = _splitk_plan(M, N, K, device)
        if split_k > 1:
            ws = _workspace(device, ws_bytes)
            return _lib.lib().b200_fp8_blockwise_scaled_mm_splitk(*args, 0, ws.data_ptr(), ws.numel(),
                                                                  _stream_ptr(device))
        return _lib.lib().b200_fp8_blockwise_scaled_mm(*args, _stream_ptr(device))


def sgl_per_token_group_quant_fp8(
    input: torch.Tensor,
    output_q: torch.Tensor,
    output_s: torch.Tensor,
    group_size: int,
    eps: float,
    fp8_min: float,
    fp8_max: float,
    scale_ue8m0: bool = False,
) -> None:
    """In place: writes e4m3 codes into `output_q` and fp32 scales into `output_s`.

    `output_s` is a 2-D view [rows, K/group]; column-major storage is inferred from
    stride(0) < stride(1) exactly as the reference does (per_token_group_quant_8bit.cu:153).
    """
    _check(input.is_cuda, "input must be a CUDA tensor")
    _check(input.is_contiguous(), "input must be contiguous")
    _check(output_q.is_cuda, "output_q must be a CUDA tensor")
    _check(output_q.is_contiguous(), "output_q must be contiguous")
    _check(input.numel() % group_size == 0, "input.numel() % group_size != 0")
    _check(output_s.dim() == 2, "output_s.dim() != 2")
    _check(input.dtype in _DT, "input must be float32, float16 or bfloat16")
    _check(output_q.dtype == FP8, "output_q must be float8_e4m3fn (int8 codes: sgl_per_token_group_quant_int8)")
    K = input.shape[-1]
    _check(K % group_size == 0, "the last dimension of input must be divisible by group_size")
    M = input.numel() // K
    if scale_ue8m0:
        # packed power-of-two scales: int32 [M, ceil(G/4)] view with rows contiguous
        # (per_token_group_quant_8bit.cu:54-61,153-156: column-major is required for this form)
        _check(output_s.dtype == torch.int32, "output_s must be int32 for UE8M0 scales")
        _check(group_size == 128, "UE8M0 scales are built for 128-wide groups")
        _check(output_s.stride(0) < output_s.stride(1) or output_s.shape[1] == 1,
               "UE8M0 scales must be column-major")
        _check(output_s.shape[0] == M and output_s.shape[1] == (K // 128 + 3) // 4 and output_s.stride(0) == 1,
               "output_s shape mismatch")
        if M == 0:
            return
        with torch.cuda.device(input.device):
            rc = _lib.lib().b200_per_token_group_quant_fp8_ue8m0(
                input.data_ptr(), _DT[input.dtype], output_q.data_ptr(), output_s.data_ptr(), M, K,
                output_s.stride(1), float(eps), float(fp8_min), float(fp8_max), _stream_ptr(input.device))
        _lib.check("sgl_per_token_group_quant_fp8", rc)
        return
    _check(output_s.dtype == torch.float32, "output_s must be float32")
    if M == 0:
        return
    _check(output_s.shape[0] == M and output_s.shape[1] == K // group_size, "output_s shape mismatch")
    with torch.cuda.device(input.device):
        rc = _lib.lib().b200_per_token_group_quant_fp8(
            input.data_ptr(), _DT[input.dtype], output_q.data_ptr(), output_s.data_ptr(),
            M, K, group_size, output_s.stride(0), output_s.stride(1),
            float(eps), float(fp8_min), float(fp8_max), _stream_ptr(input.device))
    _lib.check("sgl_per_token_group_quant_fp8", rc)


def sgl_per_token_group_quant_int8(
    input: torch.Tensor,
    output_q: torch.Tensor,
    output_s: torch.Tensor,
    group_size: int,
    eps: float,
    int8_min: float,
    int8_max: float,
) -> None:
    """In place: int8 codes into `output_q`, fp32 scales (amax / int8_max) into `output_s`; the clamped quotient is
    truncated toward zero (sgl-kernel/python/sgl_kernel/gemm.py:115-126;
    sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:110-111,206-207,219-228).  `output_s` is a 2-D view
    [rows, K/group], row- or column-major as for the FP8 operator."""
    _check(input.is_cuda, "input must be a CUDA tensor")
    _check(input.is_contiguous(), "input must be contiguous")
    _check(output_q.is_cuda, "output_q must be a CUDA tensor")
    _check(output_q.is_contiguous(), "output_q must be contiguous")
    _check(output_q.dtype == torch.int8, "output_q must be int8")
    _check(input.numel() % group_size == 0, "input.numel() % group_size != 0")
    _check(output_s.dim() == 2, "output_s.dim() != 2")
    _check(output_s.dtype == torch.float32, "output_s must be float32")
    _check(input.dtype in _DT, "input must be float32, float16 or bfloat16")
    K = input.shape[-1]
    _check(K % group_size == 0, "the last dimension of input must be divisible by group_size")
    M = input.numel() // K
    if M == 0:
        return
    _check(output_s.shape[0] == M and output_s.shape[1] == K // group_size, "output_s shape mismatch")
    with torch.cuda.device(input.device):
        rc = _lib.lib().b200_per_token_group_quant_int8(
            input.data_ptr(), _DT[input.dtype], output_q.data_ptr(), output_s.data_ptr(),
            M, K, group_size, output_s.stride(0), output_s.stride(1),
            float(eps), float(int8_min), float(int8_max), _stream_ptr(input.device))
    _lib.check("sgl_per_token_group_quant_int8", rc)


def fp8_blockwise_scaled_mm(
    mat_a: torch.Tensor,
    mat_b: torch.Tensor,
    scales_a: torch.Tensor,
    scales_b: torch.Tensor,
    out_dtype: torch.dtype,
    out: torch.Tensor = None,
) -> torch.Tensor:
    """mat_a [M,K] e4m3 row-major; mat_b [K,N] e4m3 column-major (= weight[N,K].T);
    scales_a [M,K/128] fp32 M-major; scales_b [K/128,N/128] fp32 K-major; returns [M,N].
    `out` (not in the reference signature): write into this [M,N] tensor (rows may be a slice of a
    larger buffer) instead of allocating."""
    _check(mat_a.is_cuda, "mat_a must be a CUDA tensor")
    _check(mat_b.is_cuda, "mat_b must be a CUDA tensor")
    _check(mat_a.dim() == 2, "mat_a must be a 2D tensor")
    _check(mat_b.dim() == 2, "mat_b must be a 2D tensor")
    _check(mat_a.stride(1) == 1, "mat_a must be a row major tensor")
    _check(mat_b.stride(0) == 1, "mat_b must be a column major tensor")
    _check(mat_a.size(1) == mat_b.size(0), "mat_a and mat_b shapes cannot be multiplied")
    _check((mat_a.size(1) * mat_a.element_size()) % 16 == 0, "mat_a must be multiple of 16 bytes for memory alignment")
    _check((mat_b.size(0) * mat_b.element_size()) % 16 == 0, "mat_b must be multiple of 16 bytes for memory alignment")
    _check(mat_a.dtype == FP8, "mat_a must be Float8_e4m3fn")
    _check(mat_b.dtype == FP8, "mat_b must be Float8_e4m3fn")
    _check(out_dtype in (torch.half, torch.bfloat16), "out_dtype must be Half or BFloat16")
    M, K = mat_a.shape
    N = mat_b.size(1)
    _check(scales_a.dim() == 2 and scales_b.dim() == 2, "scales must be 2D tensors")
    _check(M == scales_a.size(0), "size of scales_a is not matched")
    _check(K // 128 == scales_a.size(1), "size of scales_a is not matched")
    _check(scales_a.stride(0) == 1 or _is_contiguous_vector(scales_a), "scales_a must be M major")
    _check(K // 128 == scales_b.size(0), "size of scales_b is not matched")
    _check(N // 128 == scales_b.size(1), "size of scales_b is not matched")
    _check(scales_b.stride(0) == 1 or _is_contiguous_vector(scales_b), "scales_b must be K major")
    _check(scales_a.dtype == torch.float32, "scales_a must be Float32")
    _check(scales_b.dtype == torch.float32, "scales_b must be Float32")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=mat_a.device)
    else:
        _check(out.shape == (M, N) and out.dtype == out_dtype and out.stride(1) == 1 and out.is_cuda,
               "out must be a row-major [M,N] CUDA tensor of out_dtype")
    _check((N * out.element_size()) % 16 == 0, "out must be multiple of 16 bytes for memory alignment")
    _check(K % 128 == 0 and N % 128 == 0, "K and N must be multiples of 128 (block scale granularity)")
    if M == 0:
        return out
    args = (mat_a.data_ptr(), mat_a.stride(0), mat_b.data_ptr(), mat_b.stride(1),
            scales_a.data_ptr(), scales_a.stride(0), scales_a.stride(1),
            scales_b.data_ptr(), scales_b.stride(1), scales_b.stride(0),
            out.data_ptr(), out.stride(0), _DT[out_dtype], M, N, K)
    rc = launch_dense_mm(args, M, N, K, mat_a.device)
    _lib.check("fp8_blockwise_scaled_mm", rc)
    return out

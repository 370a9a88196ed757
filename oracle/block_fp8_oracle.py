"""CPU oracle for the W8A8 block-FP8 linear path.  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import
this module; the product package never does.

Every function restates, in plain torch-on-CPU arithmetic, one piece of the
reference (paths are relative to the reference checkout):

* ``quant_group_fp8_cuda_semantics``  -- the arithmetic of the CUDA kernel
  ``per_token_group_quant_8bit_kernel``
  (sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:19-114): this is the
  bit-exact target for the quantisation kernel.
* ``native_per_token_group_quant_fp8`` -- the torch twin used by the
  reference's own tests (python/sglang/test/test_block_fp8.py:24-49).
* ``native_w8a8_block_fp8_matmul``    -- python/sglang/test/test_block_fp8.py:274-326.
* ``baseline_scaled_mm``              -- sgl-kernel/tests/test_fp8_blockwise_gemm.py:19-58.
* ``per_block_cast_to_fp8`` / ``per_token_cast_to_fp8`` / ``calc_diff``
                                      -- sgl-kernel/tests/test_fp8_blockwise_moe.py:29-64.
* ``silu_and_mul``                    -- python/sglang/srt/layers/activation.py:60-62.
* ``fused_topk_native``               -- python/sglang/srt/layers/moe/topk.py:284-302.
* ``prepare_moe_input`` / ``shuffle_rows`` / ``apply_shuffle_mul_sum``
                                      -- sgl-kernel/csrc/moe/prepare_moe_input.cu:13-92,169-197,258-321.
* ``cutlass_fused_experts_fp8``       -- python/sglang/srt/layers/moe/cutlass_moe.py:29-222
  (the op sequence, with bf16 rounding at the same points).
* ``torch_w8a8_block_fp8_moe``        -- python/sglang/test/test_block_fp8.py:419-450.

Pinning: tests/golden/*.npz hold outputs of the reference's own functions
(executed from the reference checkout by tests/golden/make_golden.py); the
CPU tests check this module against them, and against the known-answer
generators of test/srt/quant/test_fp8_kernel.py:24-87.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
FP8_MIN = -448.0


# --------------------------------------------------------------------------------------
# quantisation
# --------------------------------------------------------------------------------------
def quant_group_fp8_cuda_semantics(
    x: torch.Tensor, group_size: int = 128, eps: float = 1e-10,
    fp8_min: float = FP8_MIN, fp8_max: float = FP8_MAX,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Arithmetic of the reference CUDA kernel (per_token_group_quant_8bit.cu:45-111).

    amax = max(eps, max|float(x)|)  (fp32, eps is the fp32 initial value, :45,:79)
    s    = amax / fp8_max           (IEEE fp32 divide, :86)
    q    = e4m3_rne_sat(fminf(fmaxf(float(x) / s, fp8_min), fp8_max))   (:109-111)

    NaN inputs: CUDA fmaxf/fminf return the non-NaN operand, so a NaN element
    does not poison amax and quantises to fp8_min; mirrored here.
    Returns (codes e4m3 [..,K], scales fp32 [..,K/group] row-major).
    """
    assert x.shape[-1] % group_size == 0
    xf = x.detach().to("cpu").to(torch.float32).reshape(-1, group_size)
    absx = torch.nan_to_num(xf.abs(), nan=0.0, posinf=float("inf"))
    amax = torch.clamp(absx.amax(dim=-1, keepdim=True), min=torch.tensor(eps, dtype=torch.float32))
    s = amax / torch.tensor(fp8_max, dtype=torch.float32)
    y = xf / s
    # fmaxf(NaN, lo) = lo ; then fminf(lo, hi) = lo
    y = torch.where(torch.isnan(y), torch.full_like(y, fp8_min), y)
    y = y.clamp(min=fp8_min, max=fp8_max)
    q = y.to(FP8).reshape(x.shape)
    s = s.reshape(x.shape[:-1] + (x.shape[-1] // group_size,))
    return q, s


def quant_group_int8_cuda_semantics(
    x: torch.Tensor, group_size: int = 128, eps: float = 1e-10, int8_min: float = -128.0, int8_max: float = 127.0,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """The same kernel with an int8 destination (per_token_group_quant_8bit.cu:79-111 with DST_DTYPE = int8_t,
    launched at :206-207; entry sgl_per_token_group_quant_int8 :219-228).

    amax = max(eps, max|float(x)|);  s = amax / int8_max (IEEE fp32);
    q    = (int8) trunc(fminf(fmaxf(float(x) / s, int8_min), int8_max))   -- the C++ cast truncates toward zero.
    NaN elements become int8_min, as in the FP8 form.  Returns (int8 codes [.., K], fp32 scales [.., K/group]).
    """
    assert x.shape[-1] % group_size == 0
    xf = x.detach().to("cpu").to(torch.float32).reshape(-1, group_size)
    absx = torch.nan_to_num(xf.abs(), nan=0.0, posinf=float("inf"))
    amax = torch.clamp(absx.amax(dim=-1, keepdim=True), min=torch.tensor(eps, dtype=torch.float32))
    s = amax / torch.tensor(int8_max, dtype=torch.float32)
    y = xf / s
    y = torch.where(torch.isnan(y), torch.full_like(y, int8_min), y)
    y = y.clamp(min=int8_min, max=int8_max)
    q = torch.trunc(y).to(torch.int8).reshape(x.shape)
    return q, s.reshape(x.shape[:-1] + (x.shape[-1] // group_size,))


def native_per_token_group_quant_fp8(x, group_size, eps=1e-10, dtype=FP8):
    """Torch twin from the reference tests (test_block_fp8.py:24-49).

    Differs from the CUDA kernel only for all-zero groups (eps is clamped in
    the input dtype) and NaN inputs.
    """
    assert x.shape[-1] % group_size == 0
    assert x.is_contiguous()
    finfo = torch.finfo(dtype)
    x_ = x.reshape(x.numel() // group_size, group_size)
    amax = x_.abs().max(dim=-1, keepdim=True)[0].clamp(min=eps).to(torch.float32)
    x_s = amax / finfo.max
    x_q = (x_ / x_s).clamp(min=finfo.min, max=finfo.max).to(dtype)
    return x_q.reshape(x.shape), x_s.reshape(x.shape[:-1] + (x.shape[-1] // group_size,))


def ceil_to_ue8m0(x: torch.Tensor) -> torch.Tensor:
    """2 ** ceil(log2(|x|)) in fp32 (python/sglang/test/test_block_fp8_deep_gemm_blackwell.py:48-50;
    the CUDA kernel's exp2f(ceilf(log2f(.))), per_token_group_quant_8bit.cu:87-89)."""
    return torch.pow(2.0, torch.ceil(torch.log2(x.abs())))


def quant_group_fp8_ue8m0_cuda_semantics(x: torch.Tensor, group_size: int = 128, eps: float = 1e-10):
    """The scale_ue8m0 = true arithmetic of per_token_group_quant_8bit.cu:45,86-97,110-111:
    amax = max(eps, max|x|); s = 2 ** ceil(log2(max(amax / 448, 1e-10))); q = e4m3(clamp(x / s));
    byte = int(log2(s)) + 127.  Returns (codes [M, K], scales fp32 [M, G], packed int32 [M, ceil(G/4)]
    with group g of a row in byte g % 4 of word g // 4, missing groups zero)."""
    M, K = x.shape
    G = K // group_size
    xf = x.to(torch.float32).reshape(M, G, group_size)
    amax = xf.abs().amax(dim=-1).clamp_min(eps)
    s = ceil_to_ue8m0((amax / 448.0).clamp_min(1e-10))
    q = (xf / s.unsqueeze(-1)).clamp(-448.0, 448.0).to(FP8).reshape(M, K)
    expo = torch.log2(s).to(torch.int32) + 127
    words = (G + 3) // 4
    padded = torch.zeros(M, words * 4, dtype=torch.int32)
    padded[:, :G] = expo & 0xFF
    p4 = padded.reshape(M, words, 4)
    packed = p4[..., 0] | (p4[..., 1] << 8) | (p4[..., 2] << 16) | (p4[..., 3] << 24)
    return q, s, packed.to(torch.int32)


def per_token_group_quant_mxfp8(x: torch.Tensor):
    """The reference test's power-of-two token quantiser (test_block_fp8_deep_gemm_blackwell.py:53-59):
    amax clamped at 1e-4, multiplication by the (exact) reciprocal of the power-of-two scale."""
    m, n = x.shape
    xv = x.view(m, -1, 128)
    amax = xv.abs().float().amax(dim=2).view(m, -1).clamp(1e-4)
    sf = ceil_to_ue8m0(amax / 448.0)
    return (xv * (1.0 / sf.unsqueeze(2))).to(FP8).view(m, n), sf


def per_block_quant_mxfp8(x: torch.Tensor):
    """128 x 128 weight blocks with power-of-two scales (test_block_fp8_deep_gemm_blackwell.py:62-76)."""
    m, n = x.shape
    pm, pn = (m + 127) // 128 * 128, (n + 127) // 128 * 128
    xp = torch.zeros((pm, pn), dtype=x.dtype)
    xp[:m, :n] = x
    xv = xp.view(-1, 128, pn // 128, 128)
    amax = xv.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    sf = ceil_to_ue8m0(amax / 448.0)
    xs = (xv * (1.0 / sf)).to(FP8)
    return xs.view_as(xp)[:m, :n].contiguous(), sf.view(xv.size(0), xv.size(2))


def scale_layout(s_row_major: torch.Tensor, layout: str) -> torch.Tensor:
    """Re-lay a row-major [M,G] scale matrix into one of the reference's layouts
    (python/sglang/srt/layers/quantization/fp8_kernel.py:300-341).

    "row"          -> contiguous [M,G]
    "col"          -> storage [G,M], returned as the [M,G] view with strides (1,M)
    "col_tma"      -> storage [G,align4(M)], view [:M] with strides (1,align4(M));
                      padding rows hold NaN so tests can see they were not needed
    """
    M, G = s_row_major.shape
    if layout == "row":
        return s_row_major.contiguous()
    if layout == "col":
        return s_row_major.t().contiguous().t()
    if layout == "col_tma":
        Ma = (M + 3) // 4 * 4
        buf = torch.full((G, Ma), float("nan"), dtype=s_row_major.dtype)
        buf[:, :M] = s_row_major.t()
        return buf.t()[:M, :]
    raise ValueError(layout)


def per_token_cast_to_fp8(x: torch.Tensor):
    """sgl-kernel/tests/test_fp8_blockwise_moe.py:40-48."""
    assert x.dim() == 2
    m, n = x.shape
    pad = (128 - (n % 128)) % 128
    x = F.pad(x, (0, pad), value=0) if pad > 0 else x
    xv = x.view(m, -1, 128)
    amax = xv.abs().float().amax(dim=2).view(m, -1).clamp(1e-4)
    q = (xv * (448.0 / amax.unsqueeze(2))).to(FP8)
    return q.view(m, n + pad)[:, :n], (amax / 448.0).view(m, -1)


def per_block_cast_to_fp8(x: torch.Tensor):
    """128x128 block quantisation of a weight matrix
    (sgl-kernel/tests/test_fp8_blockwise_moe.py:51-64)."""
    assert x.dim() == 2
    m, n = x.shape
    mp, np_ = (m + 127) // 128 * 128, (n + 127) // 128 * 128
    xp = torch.zeros((mp, np_), dtype=x.dtype)
    xp[:m, :n] = x
    xv = xp.view(-1, 128, np_ // 128, 128)
    amax = xv.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    q = (xv * (448.0 / amax)).to(FP8)
    return q.view_as(xp)[:m, :n].contiguous(), (amax / 448.0).view(xv.size(0), xv.size(2))


# --------------------------------------------------------------------------------------
# block-scaled matmul
# --------------------------------------------------------------------------------------
def block_fp8_matmul_fp32(A, B, As, Bs, block_size=(128, 128)) -> torch.Tensor:
    """fp32 result of the block-scaled product (test_block_fp8.py:274-323 before the cast).

    A [M,K] e4m3, B [N,K] e4m3, As [M,ceil(K/bk)] fp32, Bs [ceil(N/bn),ceil(K/bk)] fp32.
    C[m,n] = sum_kb (A_kb @ B_kb^T)[m,n] * (As[m,kb] * Bs[n//bn,kb]), accumulated
    kb-ascending in fp32 -- the same order and association as the reference loop.
    """
    A = A.to(torch.float32)
    B = B.to(torch.float32)
    bn, bk = block_size
    M, K = A.reshape(-1, A.shape[-1]).shape
    A = A.reshape(M, K)
    As = As.reshape(M, -1).to(torch.float32)
    N = B.shape[0]
    kt = (K + bk - 1) // bk
    nt = (N + bn - 1) // bn
    assert As.shape[1] == kt and tuple(Bs.shape) == (nt, kt)
    C = torch.zeros((M, N), dtype=torch.float32)
    Bs_rows = Bs.to(torch.float32).repeat_interleave(bn, dim=0)[:N]  # [N, kt]
    for i in range(kt):
        a = A[:, i * bk:min((i + 1) * bk, K)]
        b = B[:, i * bk:min((i + 1) * bk, K)]
        s = As[:, i:i + 1] * Bs_rows[:, i][None, :]
        C += torch.matmul(a, b.t()) * s
    return C


def native_w8a8_block_fp8_matmul(A, B, As, Bs, block_size, output_dtype=torch.float16):
    """test_block_fp8.py:274-326 (fp32 accumulate, one cast at the end)."""
    C = block_fp8_matmul_fp32(A, B, As, Bs, block_size)
    return C.reshape(A.shape[:-1] + (B.shape[0],)).to(output_dtype)


def baseline_scaled_mm(a, b, scale_a, scale_b, out_dtype, bias=None):
    """sgl-kernel/tests/test_fp8_blockwise_gemm.py:19-58: broadcast the group
    scales to full size, scale both operands in fp32, one fp32 mm, cast.
    a [M,K], b [K,N] (any strides), scale_a [M,K/128], scale_b [K/128,N/128]."""
    def group_broadcast(t, shape):
        for i, s in enumerate(shape):
            if t.shape[i] != s and t.shape[i] != 1:
                assert s % t.shape[i] == 0
                t = (t.unsqueeze(i + 1)
                     .expand(*t.shape[:i + 1], s // t.shape[i], *t.shape[i + 1:])
                     .flatten(i, i + 1))
        return t
    sa = group_broadcast(scale_a, a.shape)
    sb = group_broadcast(scale_b, b.shape)
    out = torch.mm(sa * a.to(torch.float32), sb * b.to(torch.float32)).to(out_dtype)
    if bias is not None:
        out = out + bias
    return out


def calc_diff(x, y) -> float:
    """DeepGEMM-style similarity gap (sgl-kernel/tests/test_fp8_blockwise_moe.py:29-33)."""
    x, y = x.double(), y.double()
    return float(1 - 2 * (x * y).sum() / (x * x + y * y).sum())


def rel_l2(x, ref) -> float:
    x, ref = x.double(), ref.double()
    return float((x - ref).norm() / ref.norm().clamp_min(1e-300))


def mean_rel_err(x, ref) -> float:
    """Metric of test_block_fp8.py:394-398."""
    x, ref = x.to(torch.float32), ref.to(torch.float32)
    return float((x - ref).abs().mean() / ref.abs().mean())


def block_fp8_linear(x, w_q, w_s, bias=None, out_dtype=torch.bfloat16):
    """The glue of fp8_utils.py:182-212: view(-1,K) -> quant -> GEMM -> +bias -> view."""
    x2 = x.reshape(-1, x.shape[-1])
    q, s = quant_group_fp8_cuda_semantics(x2, 128)
    out = block_fp8_matmul_fp32(q, w_q, s, w_s).to(out_dtype)
    if bias is not None:
        out = out + bias
    return out.reshape(x.shape[:-1] + (w_q.shape[0],))


# --------------------------------------------------------------------------------------
# Producer of the linear's input
# --------------------------------------------------------------------------------------
def rmsnorm_native(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None):
    """RMSNorm.forward_native (python/sglang/srt/layers/layernorm.py:135-171): fp32 throughout --
    x (+ residual, which is returned rounded to the input type), x * rsqrt(mean(x^2) + eps), * weight -- and one
    rounding to the input type at the end.  Returns y, or (y, residual_out)."""
    orig = x.dtype
    xf = x.to(torch.float32)
    res_out = None
    if residual is not None:
        xf = xf + residual.to(torch.float32)
        res_out = xf.to(orig)
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    y = ((xf * torch.rsqrt(var + eps)) * weight).to(orig)
    return y if residual is None else (y, res_out)


# --------------------------------------------------------------------------------------
# MoE glue
# --------------------------------------------------------------------------------------
def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """activation.py:60-62, evaluated in fp32 and rounded once to x.dtype
    (what the CUDA op does: fp32 math, one store)."""
    d = x.shape[-1] // 2
    xf = x.to(torch.float32)
    return (F.silu(xf[..., :d]) * xf[..., d:]).to(x.dtype)


def fused_topk_native(gating_output: torch.Tensor, topk: int, renormalize: bool = False):
    """topk.py:284-302."""
    w = F.softmax(gating_output.float(), dim=-1)
    w, ids = torch.topk(w, topk, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, ids.to(torch.int32)


def prepare_moe_input(topk_ids: torch.Tensor, num_experts: int, n: int, k: int):
    """prepare_moe_input.cu:13-92.  Returns (expert_offsets[E+1], problem_sizes1[E,3],
    problem_sizes2[E,3], input_permutation[M*topk], output_permutation[M*topk]).

    The reference assigns slots inside an expert with atomics (order unspecified);
    this restatement uses ascending flat index, one of the orders the reference
    can produce.  ids outside [0,E) (EP-masked -1) get no slot; their
    output_permutation entry is left at -1 here (the reference leaves it unwritten).
    """
    flat = topk_ids.reshape(-1).to(torch.int64)
    topk = topk_ids.shape[1]
    counts = torch.zeros(num_experts, dtype=torch.int64)
    valid = (flat >= 0) & (flat < num_experts)
    counts.scatter_add_(0, flat[valid], torch.ones_like(flat[valid]))
    offs = torch.zeros(num_experts + 1, dtype=torch.int64)
    offs[1:] = counts.cumsum(0)
    ps1 = torch.stack([counts, torch.full_like(counts, 2 * n), torch.full_like(counts, k)], 1)
    ps2 = torch.stack([counts, torch.full_like(counts, k), torch.full_like(counts, n)], 1)
    a_map = torch.full((flat.numel(),), -1, dtype=torch.int64)
    c_map = torch.full((flat.numel(),), -1, dtype=torch.int64)
    order = torch.argsort(torch.where(valid, flat, torch.full_like(flat, num_experts)), stable=True)
    nvalid = int(valid.sum())
    order = order[:nvalid]
    a_map[:nvalid] = order // topk
    c_map[order] = torch.arange(nvalid)
    i32 = torch.int32
    return offs.to(i32), ps1.to(i32), ps2.to(i32), a_map.to(i32), c_map.to(i32)


def moe_align_block_size(topk_ids: torch.Tensor, num_slots: int, block_size: int, sorted_capacity: Optional[int] = None):
    """sgl-kernel/csrc/moe/moe_align_kernel.cu:57-216 (one-block count, padded prefix, block -> expert table) and
    :28-41 (placement), with the caller's sizing of fused_moe_triton/fused_moe.py:598-605.

    `num_slots` is what the op receives as num_experts: real experts + 1, slot = id + 1, so slot 0 collects the
    id -1 of experts filtered out under expert parallelism.  Returns (sorted_token_ids[capacity],
    expert_ids[capacity // block_size rounded up], num_tokens_post_pad, cumsum[num_slots + 1]); positions not
    holding a flat index hold numel.  Inside a slot the flat indices ascend: the reference places them with
    atomics, so any order inside a slot is a valid output of it, this is the reproducible one.  Pinned by
    the worked example in the caller's docstring (fused_moe.py:583-596, ids shifted to start at 0).
    """
    flat = topk_ids.reshape(-1).to(torch.int64)
    numel = flat.numel()
    if sorted_capacity is None:
        sorted_capacity = numel + num_slots * (block_size - 1)
    slot = flat + 1
    valid = (slot >= 0) & (slot < num_slots)
    counts = torch.zeros(num_slots, dtype=torch.int64)
    counts.scatter_add_(0, slot[valid], torch.ones_like(slot[valid]))
    padded = (counts + block_size - 1) // block_size * block_size
    cumsum = torch.zeros(num_slots + 1, dtype=torch.int64)
    cumsum[1:] = padded.cumsum(0)
    total = int(cumsum[-1])
    sorted_ids = torch.full((sorted_capacity,), numel, dtype=torch.int64)
    expert_ids = torch.zeros(((sorted_capacity + block_size - 1) // block_size,), dtype=torch.int64)
    order = torch.argsort(torch.where(valid, slot, torch.full_like(slot, num_slots)), stable=True)[: int(valid.sum())]
    within = torch.arange(order.numel()) - (counts.cumsum(0) - counts)[slot[order]]
    sorted_ids[cumsum[slot[order]] + within] = order
    for e in range(num_slots):
        expert_ids[int(cumsum[e]) // block_size: int(cumsum[e + 1]) // block_size] = e - 1
    i32 = torch.int32
    return sorted_ids.to(i32), expert_ids.to(i32), total, cumsum.to(i32)


def shuffle_rows(inp: torch.Tensor, dst2src: torch.Tensor, out_rows: Optional[int] = None):
    """prepare_moe_input.cu:169-197: out[d] = inp[dst2src[d]]."""
    idx = dst2src.to(torch.int64)
    if out_rows is not None:
        idx = idx[:out_rows]
    if inp.dtype == FP8:
        return inp.view(torch.uint8)[idx].view(FP8)
    return inp[idx]


def apply_shuffle_mul_sum(inp, permutation, factors, m: int):
    """prepare_moe_input.cu:258-321: out[i] = sum_j factor[i,j] * inp[perm[i*topk+j]],
    accumulated j-ascending in fp32 (factor is read in the io dtype), one cast at the end."""
    topk = permutation.numel() // m
    perm = permutation.to(torch.int64).reshape(m, topk)
    acc = torch.zeros((m, inp.shape[1]), dtype=torch.float32)
    for j in range(topk):
        f = 1.0 if factors is None else factors.reshape(m, topk)[:, j].to(torch.float32)[:, None]
        acc = acc + f * inp[perm[:, j]].to(torch.float32)
    return acc.to(inp.dtype)


def cutlass_fused_experts_fp8(a, w1_q, w2_q, w1_s, w2_s, topk_weights, topk_ids):
    """Op sequence of cutlass_moe.py:144-221 with natural [E,N,K] weights.

    a [M,K] bf16/fp16; w1_q [E,2n,K] e4m3; w2_q [E,K,n] e4m3; w1_s [E,2n/128,K/128];
    w2_s [E,K/128,n/128]; topk_weights [M,topk]; topk_ids [M,topk] int32.
    quant -> gather -> GEMM1 -> bf16 -> silu*mul -> bf16 -> quant -> GEMM2 -> bf16 ->
    weighted un-permute sum (fp32) -> bf16.
    """
    E = w1_q.shape[0]
    m, k = a.shape
    n = w2_q.shape[2]
    offs, _, _, a_map, c_map = prepare_moe_input(topk_ids, E, n, k)
    total = int(offs[-1])
    a_q, a_s = quant_group_fp8_cuda_semantics(a, 128)
    rep_q = shuffle_rows(a_q, a_map, total)
    rep_s = shuffle_rows(a_s, a_map, total)
    c1 = torch.zeros((total, 2 * n), dtype=a.dtype)
    for e in range(E):
        lo, hi = int(offs[e]), int(offs[e + 1])
        if hi > lo:
            c1[lo:hi] = block_fp8_matmul_fp32(rep_q[lo:hi], w1_q[e], rep_s[lo:hi], w1_s[e]).to(a.dtype)
    inter = silu_and_mul(c1)
    i_q, i_s = quant_group_fp8_cuda_semantics(inter, 128)
    c2 = torch.zeros((total, k), dtype=a.dtype)
    for e in range(E):
        lo, hi = int(offs[e]), int(offs[e + 1])
        if hi > lo:
            c2[lo:hi] = block_fp8_matmul_fp32(i_q[lo:hi], w2_q[e], i_s[lo:hi], w2_s[e]).to(a.dtype)
    # rows whose expert was masked (-1) contribute nothing
    c_map64 = c_map.to(torch.int64)
    c2p = torch.cat([c2, torch.zeros((1, k), dtype=a.dtype)], 0)
    c_map_safe = torch.where(c_map64 < 0, torch.full_like(c_map64, total), c_map64)
    return apply_shuffle_mul_sum(c2p, c_map_safe, topk_weights.to(a.dtype), m)


def torch_w8a8_block_fp8_moe(a, w1, w2, w1_s, w2_s, score, topk, block_shape=(128, 128)):
    """test_block_fp8.py:419-450 (router softmax+topk inside, no renormalisation)."""
    B, D = a.shape
    a_rep = a.view(B, -1, D).repeat(1, topk, 1).reshape(-1, D)
    out = torch.zeros(B * topk, w2.shape[1], dtype=a.dtype)
    score = torch.softmax(score, dim=-1, dtype=torch.float32)
    topk_weight, topk_ids = torch.topk(score, topk)
    topk_weight = topk_weight.view(-1)
    topk_ids = topk_ids.view(-1)
    bk = block_shape[1]
    a_q, a_s = native_per_token_group_quant_fp8(a_rep, bk)
    a_q = a_q.to(torch.float32)
    for i in range(w1.shape[0]):
        mask = topk_ids == i
        if mask.sum():
            inter = native_w8a8_block_fp8_matmul(a_q[mask], w1[i], a_s[mask], w1_s[i], block_shape, a.dtype)
            d = inter.shape[-1] // 2
            act = F.silu(inter[..., :d]) * inter[..., d:]
            act_q, act_s = native_per_token_group_quant_fp8(act, bk)
            out[mask] = native_w8a8_block_fp8_matmul(act_q, w2[i], act_s, w2_s[i], block_shape, a.dtype)
    return (out.view(B, -1, w2.shape[1]) * topk_weight.view(B, -1, 1).to(out.dtype)).sum(dim=1)


# --------------------------------------------------------------------------------------
# seeded synthetic inputs (shapes of the benchmark configurations)
# --------------------------------------------------------------------------------------
def gen_activation(M: int, K: int, seed: int, dtype=torch.bfloat16, outlier_frac: float = 0.0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((M, K), generator=g, dtype=torch.float32)
    if outlier_frac > 0:
        mask = torch.rand((M, K), generator=g) < outlier_frac
        x = torch.where(mask, x * 100.0, x)
    return x.to(dtype)


def gen_weight(N: int, K: int, seed: int, std: float = 0.02):
    """N(0,std^2) weight, block-quantised with per_block_cast_to_fp8."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn((N, K), generator=g, dtype=torch.float32) * std
    return per_block_cast_to_fp8(w)

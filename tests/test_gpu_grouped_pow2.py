"""GPU parity: the block-scaling (power-of-two scales) expert path -- quantisation with a fused row gather,
SiLU*mul + power-of-two quantisation, the grouped block-scaling GEMM behind DeepGEMM's contiguous and masked
call surface, and the fused expert layer built from them.

Checkers: the CPU oracle (oracle/block_fp8_oracle.py) for the arithmetic, this library's own dense entry points
where the claim is "same bits as the unfused / ungrouped sequence"."""
import pytest
import torch

from oracle import block_fp8_oracle as O
from helpers import same_bits

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn
TOL = 1e-3


def _status_ok():
    import ctypes
    from sglang_b200 import _lib
    st = ctypes.c_int(0)
    _lib.check("status", _lib.lib().b200_gemm_device_status(ctypes.byref(st)))
    assert st.value == 0, f"device status word = {st.value}"


@pytest.mark.parametrize("ue8m0", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,K,R", [(1, 128, 5), (50, 512, 333), (300, 7168, 1000)])
def test_gather_quant_equals_quant_then_gather(M, K, R, dtype, ue8m0):
    from sglang_b200.layers.quantization.fp8_kernel import (gather_per_token_group_quant_fp8,
                                                            sglang_per_token_group_quant_fp8)
    g = torch.Generator().manual_seed(M + K + R)
    x = O.gen_activation(M, K, seed=M + R, outlier_frac=1e-3).to(dtype).cuda()
    idx = torch.randint(0, M, (R,), generator=g, dtype=torch.int32).cuda()
    kw = dict(column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True) if ue8m0 else {}
    q, s = sglang_per_token_group_quant_fp8(x, 128, **kw)
    gq, gs = gather_per_token_group_quant_fp8(x, idx, 128, **kw)
    q8 = q.view(torch.uint8)
    assert torch.equal(gq.view(torch.uint8).cpu(), q8[idx.long()].cpu())
    assert torch.equal(gs.cpu(), s[idx.long()].cpu())
    # out-of-range indices are clamped into the rows of x, never followed out of the buffer
    bad = torch.tensor([-5, M + 100], dtype=torch.int32).cuda()
    bq, _ = gather_per_token_group_quant_fp8(x, bad, 128, **kw)
    assert torch.equal(bq.view(torch.uint8).cpu(), torch.stack([q8[0], q8[M - 1]]).cpu())
    eq, es = gather_per_token_group_quant_fp8(x, idx[:0], 128, **kw)
    assert eq.shape == (0, K) and es.shape[0] == 0


@pytest.mark.parametrize("M,K,R", [(1, 128, 5), (50, 512, 333), (300, 7168, 1001)])
def test_shuffle_packed_scales(M, K, R):
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    from sglang_b200.sgl_kernel import shuffle_packed_scales
    x = O.gen_activation(M, K, seed=M + R, outlier_frac=1e-3).cuda()
    idx = torch.randint(0, M, (R,), generator=torch.Generator().manual_seed(R), dtype=torch.int32).cuda()
    _, s = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
    out = shuffle_packed_scales(s, idx)
    assert out.shape == (R, s.shape[1]) and (out.stride(0) == 1 or R == 1) and out.stride(1) % 4 == 0
    assert torch.equal(out.cpu(), s[idx.long()].cpu())
    bad = torch.tensor([-3, M + 7], dtype=torch.int32).cuda()      # clamped into the source rows
    assert torch.equal(shuffle_packed_scales(s, bad).cpu(), torch.stack([s[0], s[M - 1]]).cpu())
    assert shuffle_packed_scales(s, idx[:0]).shape == (0, s.shape[1])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K", [(1, 128), (77, 2048), (300, 512)])
def test_silu_mul_quant_power_of_two_scales(M, K, dtype):
    """One pass == silu_and_mul, then the power-of-two quantisation (bits), and equal to the oracle's restatement."""
    from sglang_b200.layers.quantization.fp8_kernel import (sglang_per_token_group_quant_fp8,
                                                            silu_and_mul_per_token_group_quant_fp8)
    from sglang_b200.sgl_kernel import silu_and_mul
    g = torch.Generator().manual_seed(M * 7 + K)
    x = (torch.randn(M, 2 * K, generator=g) * 3).to(dtype).cuda()
    q, s = silu_and_mul_per_token_group_quant_fp8(x, 128, scale_ue8m0=True)
    mid = torch.empty(M, K, dtype=dtype, device="cuda")
    silu_and_mul(x, mid)
    q2, s2 = sglang_per_token_group_quant_fp8(mid, 128, column_major_scales=True, scale_tma_aligned=True,
                                              scale_ue8m0=True)
    assert same_bits(q.cpu(), q2.cpu()) and torch.equal(s.cpu(), s2.cpu())
    assert s.stride(0) == 1 or M == 1
    q_ref, _, packed_ref = O.quant_group_fp8_ue8m0_cuda_semantics(mid.cpu(), 128)
    assert same_bits(q.cpu(), q_ref) and torch.equal(s.cpu(), packed_ref)


def _make_experts(E, N, K, seed):
    """Weights whose blocks carry very different power-of-two scales, so that a scale taken from the wrong expert,
    column block or k-block cannot pass."""
    g = torch.Generator().manual_seed(seed)
    wq, ws = [], []
    for e in range(E):
        w = torch.randn(N, K, generator=g) * 0.02
        blk = (torch.arange(N // 128).unsqueeze(1) * (K // 128) + torch.arange(K // 128).unsqueeze(0) + e) % 7
        w = w * torch.pow(2.0, blk.float()).repeat_interleave(128, 0).repeat_interleave(128, 1)
        q_, s_ = O.per_block_quant_mxfp8(w)
        wq.append(q_)
        ws.append(s_)
    return torch.stack(wq), torch.stack(ws)


def _rows(R, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(R, K, generator=g)
    x = (x * torch.pow(2.0, (torch.arange(R) % 13).float()).unsqueeze(1)).to(torch.bfloat16)
    x[:, : K // 2] *= 4.0
    return x


@pytest.mark.parametrize("tile_hook", [0, 9240, 9192, 9480])      # 128 x 256 (default), 128 x 240, 128 x 192, 256 x 240 tiles
@pytest.mark.parametrize("sizes,N,K", [([5], 256, 128), ([0, 1, 127, 128, 129, 300, 0, 64], 512, 1024),
                                       ([130] * 20, 1152, 640), ([256, 3, 700], 4096, 7168)])
def test_grouped_block_scaling_gemm_problem_table(sizes, N, K, tile_hook):
    """Problems of ragged sizes packed without padding (what b200_moe_prepare writes), including empty ones: every
    expert's rows against the oracle's fp32 product and, bit for bit, against the dense block-scaling entry run on
    that expert alone; rows between problems and a skipped problem stay untouched."""
    from sglang_b200.layers.quantization.deep_gemm_wrapper import grouped_gemm_pow2
    from sglang_b200.layers.quantization.fp8_kernel import (sglang_per_token_group_quant_fp8,
                                                            w8a8_block_fp8_matmul_deepgemm)
    E = len(sizes)
    wq, ws = _make_experts(E, N, K, seed=N + K)
    gap = 3                                       # unowned rows between the problems
    offsets, R = [], 0
    for sz in sizes:
        offsets.append(R)
        R += sz + gap
    x = _rows(R, K, seed=R)
    q, sp = sglang_per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True, scale_tma_aligned=True,
                                             scale_ue8m0=True)
    q_ref, s_ref, _ = O.quant_group_fp8_ue8m0_cuda_semantics(x, 128)
    d = dict(dtype=torch.int32, device="cuda")
    off_t = torch.tensor(offsets, **d)
    ps = torch.zeros(E, 3, **d)
    ps[:, 0] = torch.tensor(sizes, **d)
    experts = torch.arange(E, **d)
    skipped = E - 1 if E > 2 else -1
    if skipped >= 0:
        experts[skipped] = -1
    from sglang_b200 import _lib
    out = torch.full((R, N), 7.0, dtype=torch.bfloat16, device="cuda")
    _lib.lib().b200_debug_force_block_n(tile_hook)
    try:
        grouped_gemm_pow2(q, sp, wq.cuda(), ws.cuda(), out, off_t, ps[:, 0], experts)
        _status_ok()
    finally:
        _lib.lib().b200_debug_force_block_n(0)
    out = out.cpu()
    owned = torch.zeros(R, dtype=torch.bool)
    for e, (o, sz) in enumerate(zip(offsets, sizes)):
        if sz == 0 or e == skipped:
            continue
        owned[o:o + sz] = True
        ref32 = O.block_fp8_matmul_fp32(q_ref[o:o + sz], wq[e], s_ref[o:o + sz], ws[e])
        assert O.rel_l2(out[o:o + sz].float(), ref32.to(torch.bfloat16).float()) <= TOL, e
        xe = x[o:o + sz].cuda().contiguous()
        qe, se = sglang_per_token_group_quant_fp8(xe, 128, column_major_scales=True, scale_tma_aligned=True,
                                                  scale_ue8m0=True)
        dense = w8a8_block_fp8_matmul_deepgemm(qe, wq[e].cuda(), se, ws[e].cuda(), [128, 128], torch.bfloat16,
                                               weight_scale_ue8m0=True)
        assert same_bits(out[o:o + sz], dense.cpu()), e
    assert (out[~owned] == 7.0).all(), "a row outside every problem was written"


def test_deepgemm_contiguous_layout():
    """entrypoint.py:62-75 as its caller uses it (ep_moe/layer.py:540-640): experts' rows padded to 128, m_indices per
    row, padding blocks marked -1."""
    from sglang_b200.layers.quantization import deep_gemm_wrapper as dg
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    E, N, K = 6, 512, 1024
    wq, ws = _make_experts(E, N, K, seed=3)
    block_expert = [4, 4, 0, -1, 2, 5, 5, 5, -1, 1]       # expert of every 128-row block
    M = 128 * len(block_expert)
    x = _rows(M, K, seed=9)
    m_indices = torch.tensor(block_expert, dtype=torch.int32).repeat_interleave(128).cuda()
    q, sp = sglang_per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True, scale_tma_aligned=True,
                                             scale_ue8m0=True)
    q_ref, s_ref, _ = O.quant_group_fp8_ue8m0_cuda_semantics(x, 128)
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    dg.grouped_gemm_nt_f8f8bf16_contig((q, sp), (wq.cuda(), ws.cuda()), out, m_indices)
    _status_ok()
    out = out.cpu()
    for b, e in enumerate(block_expert):
        rows = slice(128 * b, 128 * b + 128)
        if e < 0:
            assert (out[rows] == 7.0).all()
            continue
        ref32 = O.block_fp8_matmul_fp32(q_ref[rows], wq[e], s_ref[rows], ws[e])
        assert O.rel_l2(out[rows].float(), ref32.to(torch.bfloat16).float()) <= TOL, b
    assert dg.get_m_alignment_for_contiguous_layout() == 128


def test_deepgemm_masked_layout_and_dense_entry():
    """entrypoint.py:39-59 as its caller uses it (ep_moe/layer.py:205-320): [E, max_m, K] with masked_m valid rows per
    expert and the scales cast to packed exponents per expert (the arithmetic of _cast_to_e8m0_with_rounding_up,
    ep_moe/layer.py:62-72, restated below); and gemm_nt_f8f8bf16 (:78-93) on one expert."""
    from sglang_b200.layers.quantization import deep_gemm_wrapper as dg
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    E, max_m, N, K = 5, 192, 384, 2048
    masked = [0, 192, 1, 130, 64]
    wq, ws = _make_experts(E, N, K, seed=5)
    x = _rows(E * max_m, K, seed=11)
    q_ref, s_ref, _ = O.quant_group_fp8_ue8m0_cuda_semantics(x, 128)          # s_ref: fp32 powers of two [R, K/128]
    # fp32 scales [E, max_m, G] -> exponent bytes -> int32 words with the rows of an expert contiguous
    exp = (s_ref.view(torch.int32) >> 23).to(torch.uint8).view(E, max_m, K // 128)
    packed = exp.contiguous().view(torch.int32)                                  # [E, max_m, G/4]
    packed = packed.transpose(1, 2).contiguous().transpose(1, 2).cuda()
    assert packed.stride(1) == 1 or max_m == 1
    out = torch.full((E, max_m, N), 7.0, dtype=torch.bfloat16, device="cuda")
    masked_m = torch.tensor(masked, dtype=torch.int32).cuda()
    dg.grouped_gemm_nt_f8f8bf16_masked((q_ref.view(E, max_m, K).cuda(), packed), (wq.cuda(), ws.cuda()), out, masked_m,
                                       expected_m=128)
    _status_ok()
    out = out.cpu()
    for e, mm in enumerate(masked):
        r0 = e * max_m
        assert (out[e, mm:] == 7.0).all(), "rows past masked_m were written"
        if mm:
            ref32 = O.block_fp8_matmul_fp32(q_ref[r0:r0 + mm], wq[e], s_ref[r0:r0 + mm], ws[e])
            assert O.rel_l2(out[e, :mm].float(), ref32.to(torch.bfloat16).float()) <= TOL, e
    # dense entry
    q, sp = sglang_per_token_group_quant_fp8(x[:300].cuda().contiguous(), 128, column_major_scales=True,
                                             scale_tma_aligned=True, scale_ue8m0=True)
    o2 = torch.empty(300, N, dtype=torch.bfloat16, device="cuda")
    dg.gemm_nt_f8f8bf16((q, sp), (wq[1].cuda(), ws[1].cuda()), o2)
    ref32 = O.block_fp8_matmul_fp32(q_ref[:300], wq[1], s_ref[:300], ws[1])
    assert O.rel_l2(o2.float().cpu(), ref32.to(torch.bfloat16).float()) <= TOL
    _status_ok()


def _fp32_expert_layer_ue8m0(x, w13, w2, w13s, w2s, tw, ti):
    """fp32 restatement on the GPU of the op sequence with power-of-two activation scales: per expert quantise
    (scale = 2^ceil(log2(amax/448))), block-scaled product, bf16, SiLU*mul, quantise, product, bf16; weighted sum."""
    E, I = w13.shape[0], w2.shape[2]
    m, topk = ti.shape
    H = x.shape[1]
    dev = x.device

    def quant(t_):
        tf = t_.float().view(t_.shape[0], -1, 128)
        amax_ = tf.abs().amax(-1).clamp(min=1e-10)
        s_ = amax_ / torch.full_like(amax_, 448.0)
        s_ = torch.exp2(torch.ceil(torch.log2(s_.clamp(min=1e-10))))
        return (tf / s_.unsqueeze(-1)).clamp(-448.0, 448.0).to(FP8).view(t_.shape), s_

    def mm(a_q, w_q, sa, sw):
        K = a_q.shape[1]
        c = torch.zeros(a_q.shape[0], w_q.shape[0], device=dev)
        sw_rows = sw.repeat_interleave(128, 0)
        for kb in range(K // 128):
            c += (a_q[:, kb * 128:(kb + 1) * 128].float() @ w_q[:, kb * 128:(kb + 1) * 128].float().t()) * \
                 (sa[:, kb:kb + 1] * sw_rows[:, kb][None, :])
        return c
    xq, xs = quant(x)
    flat_e = ti.reshape(-1).long()
    flat_t = torch.arange(m, device=dev).repeat_interleave(topk)
    contrib = torch.zeros(m * topk, H, device=dev, dtype=torch.bfloat16)
    for e in range(E):
        sel = (flat_e == e).nonzero().flatten()
        if sel.numel() == 0:
            continue
        rows = flat_t[sel]
        c1 = mm(xq[rows], w13[e], xs[rows], w13s[e]).to(torch.bfloat16)
        act = (torch.nn.functional.silu(c1[:, :I].float()) * c1[:, I:].float()).to(torch.bfloat16)
        aq, as_ = quant(act)
        contrib[sel] = mm(aq, w2[e], as_, w2s[e]).to(torch.bfloat16)
    w = tw.to(torch.bfloat16).float().reshape(m, topk, 1)
    return (contrib.float().view(m, topk, H) * w).sum(1).to(torch.bfloat16)


@pytest.mark.parametrize("E,H,I,m,topk", [(8, 512, 256, 70, 2), (32, 1024, 512, 600, 4)])
def test_fused_experts_power_of_two_scales(E, H, I, m, topk):
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8_ue8m0
    old_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        w13, w13s = _make_experts(E, 2 * I, H, seed=E)
        w2, w2s = _make_experts(E, H, I, seed=E + 1)
        w13, w13s, w2, w2s = w13.cuda(), w13s.cuda(), w2.cuda(), w2s.cuda()
        g = torch.Generator().manual_seed(m)
        x = torch.randn(m, H, generator=g).to(torch.bfloat16).cuda()
        tw, ti = O.fused_topk_native(torch.randn(m, E, generator=g), topk)
        tw, ti = tw.cuda(), ti.to(torch.int32).cuda()
        out = fused_experts_block_fp8_ue8m0(x, w13, w2, w13s, w2s, tw, ti)
        assert same_bits(out, fused_experts_block_fp8_ue8m0(x, w13, w2, w13s, w2s, tw, ti)), "not deterministic"
        ref = _fp32_expert_layer_ue8m0(x, w13, w2, w13s, w2s, tw, ti)
        assert O.rel_l2(out.float().cpu(), ref.float().cpu()) <= 5e-3
        _status_ok()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old_tf32


def test_fused_experts_power_of_two_scales_full_size_256_experts_4096_tokens():
    """The MoE benchmark configuration at size (256 experts, hidden 7168, intermediate 2048, 4096 tokens, top-8) on the
    block-scaling path: every token against the fp32 restatement on the GPU."""
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8_ue8m0
    old_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        E, H, I, m, topk = 256, 7168, 2048, 4096, 8
        dev = torch.device("cuda")
        w13 = torch.empty(E, 2 * I, H, dtype=FP8, device=dev)
        w2 = torch.empty(E, H, I, dtype=FP8, device=dev)
        w13s = torch.empty(E, 2 * I // 128, H // 128, device=dev)
        w2s = torch.empty(E, H // 128, I // 128, device=dev)
        g = torch.Generator(device=dev).manual_seed(41)

        def block_quant_pow2(w):    # per_block_cast_to_fp8 with the scale rounded up to a power of two, on the device
            n, k = w.shape
            wv = w.view(n // 128, 128, k // 128, 128)
            amax = wv.abs().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
            s = torch.exp2(torch.ceil(torch.log2(amax / 448.0)))
            return (wv / s).to(FP8).view(n, k), s.view(n // 128, k // 128)
        for e in range(E):
            w13[e], w13s[e] = block_quant_pow2(torch.randn(2 * I, H, generator=g, device=dev) * 0.02)
            w2[e], w2s[e] = block_quant_pow2(torch.randn(H, I, generator=g, device=dev) * 0.02)
        x = torch.randn(m, H, generator=g, device=dev).to(torch.bfloat16)
        logits = torch.randn(m, E, generator=g, device=dev)
        tw, ti = torch.topk(torch.softmax(logits.float(), dim=-1), topk, dim=-1)
        ti = ti.to(torch.int32)
        out = fused_experts_block_fp8_ue8m0(x, w13, w2, w13s, w2s, tw, ti)
        ref = _fp32_expert_layer_ue8m0(x, w13, w2, w13s, w2s, tw, ti)
        err = O.rel_l2(out.float().cpu(), ref.float().cpu())
        assert err <= 5e-3, err
        _status_ok()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old_tf32


@pytest.mark.parametrize("M,K", [(1, 128), (37, 1024), (64, 7168), (130, 2048)])
def test_packed_exponents_with_contiguous_rows(M, K):
    """per_token_group_quant_fp8_ue8m0_rows: the codes and exponent bytes of the column-major packed form, one
    contiguous (padded) row of words per token."""
    from sglang_b200.layers.quantization.fp8_kernel import (per_token_group_quant_fp8_ue8m0_rows,
                                                            sglang_per_token_group_quant_fp8)
    x = O.gen_activation(M, K, seed=M + K, outlier_frac=1e-3).cuda()
    q, s = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
    q2, s2 = per_token_group_quant_fp8_ue8m0_rows(x)
    W = s.shape[1]
    assert s2.is_contiguous() and s2.shape[1] % 4 == 0 and s2.shape[1] >= W
    assert same_bits(q2.cpu(), q.cpu()) and torch.equal(s2[:, :W].cpu(), s.cpu()) and (s2[:, W:] == 0).all()


def test_prequantized_rows_on_the_block_scaling_path_equal_the_fused_layer():
    """What an expert-parallel rank runs on received rows (codes + contiguous exponent words + local expert ids, some
    rows empty) against the single-GPU layer on the same routing: same bits, row by row."""
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8_ue8m0, grouped_experts_prequantized_ue8m0
    from sglang_b200.layers.quantization.fp8_kernel import per_token_group_quant_fp8_ue8m0_rows
    E, H, I, m = 8, 512, 256, 70
    w13, w13s = _make_experts(E, 2 * I, H, seed=21)
    w2, w2s = _make_experts(E, H, I, seed=22)
    w13, w13s, w2, w2s = w13.cuda(), w13s.cuda(), w2.cuda(), w2s.cuda()
    g = torch.Generator().manual_seed(5)
    x = torch.randn(m, H, generator=g).to(torch.bfloat16).cuda()
    ids = torch.randint(0, E, (m, 1), generator=g, dtype=torch.int32).cuda()
    ones = torch.ones(m, 1, device="cuda")
    ref = fused_experts_block_fp8_ue8m0(x, w13, w2, w13s, w2s, ones, ids)            # top-1, weight 1: the expert output
    q, words = per_token_group_quant_fp8_ue8m0_rows(x)
    # interleave empty rows (id -1), as a receive region with spare capacity has them
    R = 2 * m
    q_pad = torch.zeros(R, H, dtype=torch.uint8, device="cuda")
    q_pad[::2] = q.view(torch.uint8)
    w_pad = torch.zeros(R, words.shape[1], dtype=torch.int32, device="cuda")
    w_pad[::2] = words
    id_pad = torch.full((R,), -1, dtype=torch.int32, device="cuda")
    id_pad[::2] = ids.flatten()
    out = grouped_experts_prequantized_ue8m0(q_pad.view(FP8), w_pad, id_pad, w13, w2, w13s, w2s, torch.bfloat16)
    assert same_bits(out[::2].cpu(), ref.cpu())
    _status_ok()


@pytest.mark.parametrize("mid_dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("sizes,I,K", [([5], 128, 128), ([0, 1, 127, 128, 129, 300, 0, 64], 256, 1024),
                                       ([130] * 12, 640, 512), ([256, 3, 200], 2048, 7168)])
def test_gemm_epilogue_that_emits_codes_and_exponents(sizes, I, K, mid_dtype):
    """Expert GEMM 1 with SiLU*mul and the next quantisation in its epilogue against the three-kernel sequence
    (grouped GEMM into a 16-bit tensor, SiLU*mul + power-of-two quantisation): codes and exponent bytes of every owned
    row bit for bit; rows outside every problem untouched."""
    from sglang_b200.layers.quantization.deep_gemm_wrapper import grouped_gemm_pow2, grouped_gemm_pow2_silu_quant
    from sglang_b200.layers.quantization.fp8_kernel import (sglang_per_token_group_quant_fp8,
                                                            silu_and_mul_per_token_group_quant_fp8)
    E = len(sizes)
    wq, ws = _make_experts(E, 2 * I, K, seed=I + K)
    gap = 3
    offsets, R = [], 0
    for sz in sizes:
        offsets.append(R)
        R += sz + gap
    x = _rows(R, K, seed=R + 1)
    q, sp = sglang_per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True, scale_tma_aligned=True,
                                             scale_ue8m0=True)
    d = dict(dtype=torch.int32, device="cuda")
    off_t = torch.tensor(offsets, **d)
    rows_t = torch.tensor(sizes, **d)
    c1 = torch.zeros((R, 2 * I), dtype=mid_dtype, device="cuda")
    grouped_gemm_pow2(q, sp, wq.cuda(), ws.cuda(), c1, off_t, rows_t)
    q_ref, s_ref = silu_and_mul_per_token_group_quant_fp8(c1, 128, scale_ue8m0=True)
    q_f, s_f = grouped_gemm_pow2_silu_quant(q, sp, wq.cuda(), ws.cuda(), off_t, rows_t, mid_dtype=mid_dtype)
    _status_ok()
    assert s_f.shape == s_ref.shape and s_f.stride() == s_ref.stride()
    owned = torch.zeros(R, dtype=torch.bool)
    for o, sz in zip(offsets, sizes):
        owned[o:o + sz] = True
    assert owned.any()
    assert torch.equal(q_f.view(torch.uint8).cpu()[owned], q_ref.view(torch.uint8).cpu()[owned])
    assert torch.equal(s_f.cpu()[owned], s_ref.cpu()[owned])
    assert (s_f.cpu()[~owned] == 0).all(), "an exponent of a row outside every problem was written"


def test_fused_experts_with_and_without_the_activation_in_the_epilogue():
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8_ue8m0
    E, H, I, m, topk = 32, 1024, 512, 600, 4
    w13, w13s = _make_experts(E, 2 * I, H, seed=E)
    w2, w2s = _make_experts(E, H, I, seed=E + 1)
    w13, w13s, w2, w2s = w13.cuda(), w13s.cuda(), w2.cuda(), w2s.cuda()
    g = torch.Generator().manual_seed(m)
    x = torch.randn(m, H, generator=g).to(torch.bfloat16).cuda()
    tw, ti = O.fused_topk_native(torch.randn(m, E, generator=g), topk)
    tw, ti = tw.cuda(), ti.to(torch.int32).cuda()
    a = fused_experts_block_fp8_ue8m0(x, w13, w2, w13s, w2s, tw, ti, fuse_activation=True)
    b = fused_experts_block_fp8_ue8m0(x, w13, w2, w13s, w2s, tw, ti, fuse_activation=False)
    assert same_bits(a, b)
    _status_ok()


def test_dense_gate_up_with_the_activation_in_the_epilogue():
    """The dense MLP's gate_up projection + SiLU*mul + quantisation in one kernel against the three-kernel chain, and
    the chain's end (down projection) against the oracle."""
    from sglang_b200.layers.quantization.deep_gemm_wrapper import gate_up_silu_quant_pow2
    from sglang_b200.layers.quantization.fp8_kernel import (sglang_per_token_group_quant_fp8,
                                                            silu_and_mul_per_token_group_quant_fp8,
                                                            w8a8_block_fp8_matmul_deepgemm)
    M, K, I = 300, 1024, 768
    wq, ws = _make_experts(1, 2 * I, K, seed=77)
    wq, ws = wq[0].cuda(), ws[0].cuda()
    x = _rows(M, K, seed=78).cuda()
    q, sp = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
    c1 = w8a8_block_fp8_matmul_deepgemm(q, wq, sp, ws, [128, 128], torch.bfloat16, weight_scale_ue8m0=True)
    q_ref, s_ref = silu_and_mul_per_token_group_quant_fp8(c1, 128, scale_ue8m0=True)
    q_f, s_f = gate_up_silu_quant_pow2(q, sp, wq, ws)
    _status_ok()
    assert same_bits(q_f.cpu(), q_ref.cpu()) and torch.equal(s_f.cpu(), s_ref.cpu())

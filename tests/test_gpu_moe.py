"""GPU parity: MoE glue kernels and the grouped block-FP8 GEMM against the CPU oracle.

Shapes follow sgl-kernel/tests/test_fp8_blockwise_moe.py (random m_g = 16*U{1..64}, n,k multiples
of 128), python/sglang/test/test_block_fp8.py:452-525 and the DeepSeek-V3 MoE configuration at
reduced token count."""
import pytest
import torch

from oracle import block_fp8_oracle as O
from helpers import as_bf16, as_fp8, load_golden, same_bits, t

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _status_ok():
    import ctypes
    from sglang_b200 import _lib
    st = ctypes.c_int(0)
    _lib.check("status", _lib.lib().b200_gemm_device_status(ctypes.byref(st)))
    assert st.value == 0, f"device status word = {st.value}"


@pytest.mark.parametrize("m,topk,E", [(1, 1, 4), (37, 2, 8), (4096, 8, 256), (3000, 6, 64)])
def test_prepare_moe_input_exact(m, topk, E):
    from sglang_b200.sgl_kernel import prepare_moe_input
    g = torch.Generator().manual_seed(m + E)
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(m)]).to(torch.int32)
    if m > 30:
        ids[5, 0] = -1                                   # a masked (non-local) expert id
    n, k = 2048, 7168
    offs_r, ps1_r, ps2_r, a_map_r, c_map_r = O.prepare_moe_input(ids, E, n, k)
    d = dict(dtype=torch.int32, device="cuda")
    offs, ps1, ps2 = torch.empty(E + 1, **d), torch.empty(E, 3, **d), torch.empty(E, 3, **d)
    a_map, c_map = torch.full((m * topk,), -7, **d), torch.full((m * topk,), -7, **d)
    prepare_moe_input(ids.cuda(), offs, ps1, ps2, a_map, c_map, E, n, k)
    total = int(offs_r[-1])
    assert torch.equal(offs.cpu(), offs_r) and torch.equal(ps1.cpu(), ps1_r) and torch.equal(ps2.cpu(), ps2_r)
    assert torch.equal(a_map.cpu()[:total], a_map_r[:total])     # same deterministic order as the oracle
    assert torch.equal(c_map.cpu(), c_map_r)
    # twice -> identical (no atomics in the slot assignment)
    a2, c2 = torch.empty_like(a_map), torch.empty_like(c_map)
    prepare_moe_input(ids.cuda(), offs, ps1, ps2, a2, c2, E, n, k)
    assert torch.equal(a2[:total], a_map[:total]) and torch.equal(c2, c_map)


@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float32, torch.bfloat16])
def test_shuffle_rows(dtype):
    from sglang_b200.sgl_kernel import shuffle_rows
    g = torch.Generator().manual_seed(1)
    src = torch.randn(50, 256, generator=g).to(dtype)
    idx = torch.randint(0, 50, (333,), generator=g, dtype=torch.int32)
    out = shuffle_rows(src.cuda(), idx.cuda(), (333, 256))
    assert same_bits(out.cpu(), O.shuffle_rows(src, idx))
    assert shuffle_rows(src.cuda(), idx[:0].cuda(), (0, 256)).shape == (0, 256)


def test_silu_and_mul_and_weighted_sum():
    from sglang_b200.sgl_kernel import apply_shuffle_mul_sum, silu_and_mul
    g = torch.Generator().manual_seed(2)
    x = (torch.randn(77, 512, generator=g) * 3).to(torch.bfloat16)
    out = silu_and_mul(x.cuda()).cpu()
    ref = O.silu_and_mul(x)
    assert O.rel_l2(out.float(), ref.float()) < 2e-3      # __expf vs exact exp, then one bf16 rounding
    m, topk, k = 19, 4, 256
    c2 = torch.randn(m * topk, k, generator=g).to(torch.bfloat16)
    perm = torch.randperm(m * topk, generator=g).to(torch.int32)
    w = torch.rand(m, topk, generator=g).to(torch.bfloat16)
    res = torch.empty(m, k, dtype=torch.bfloat16, device="cuda")
    apply_shuffle_mul_sum(c2.cuda(), res, perm.cuda(), w.cuda())
    ref = O.apply_shuffle_mul_sum(c2, perm, w, m)
    assert O.rel_l2(res.cpu().float(), ref.float()) < 2e-3
    res1 = torch.empty(m, k, dtype=torch.bfloat16, device="cuda")
    apply_shuffle_mul_sum(c2.cuda(), res1, perm.cuda(), None)
    assert O.rel_l2(res1.cpu().float(), O.apply_shuffle_mul_sum(c2, perm, None, m).float()) < 2e-3


def _grouped_problem(E, N, K, counts, seed):
    g = torch.Generator().manual_seed(seed)
    rows = int(sum(counts))
    x = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    a, sa = O.quant_group_fp8_cuda_semantics(x, 128)
    wq, ws = [], []
    for e in range(E):
        q_, s_ = O.per_block_cast_to_fp8(torch.randn(N, K, generator=g) * 0.02)
        wq.append(q_); ws.append(s_)
    offs = torch.zeros(E + 1, dtype=torch.int32)
    offs[1:] = torch.tensor(counts).cumsum(0)
    ps = torch.tensor([[c, N, K] for c in counts], dtype=torch.int32)
    return a, sa, torch.stack(wq), torch.stack(ws), offs, ps


@pytest.mark.parametrize("kernel", [0, 3, 3032, 3064, 3128])   # 0 = automatic; 3xxx = weight-streaming kernel
@pytest.mark.parametrize("E,N,K,seed", [(4, 256, 512, 0), (8, 384, 256, 1), (16, 512, 1024, 2), (8, 4096, 7168, 3)])
def test_grouped_gemm(E, N, K, seed, kernel):
    from sglang_b200 import _lib
    from sglang_b200.sgl_kernel import fp8_blockwise_scaled_grouped_mm
    g = torch.Generator().manual_seed(100 + seed)
    counts = [int(c) for c in torch.randint(0, 5, (E,), generator=g) * 50 + torch.randint(0, 30, (E,), generator=g)]
    counts[0] = 0 if E > 4 else counts[0]                        # an expert without tokens
    counts[-1] = 130                                             # one m-tile boundary case
    a, sa, wq, ws, offs, ps = _grouped_problem(E, N, K, counts, seed)
    rows = a.shape[0]
    out = torch.full((rows + 3, N), -7.0, dtype=torch.bfloat16, device="cuda")
    _lib.lib().b200_debug_force_block_n(kernel)
    try:
        fp8_blockwise_scaled_grouped_mm(out[:rows], None, None, None, None, None, a.cuda(), wq.cuda().transpose(1, 2),
                                        sa.cuda(), ws.cuda(), None, None, None, None, None, ps.cuda(),
                                        offs[:-1].cuda(), None)
        torch.cuda.synchronize()
    finally:
        _lib.lib().b200_debug_force_block_n(0)
    _status_ok()
    assert torch.all(out[rows:] == -7.0)
    for e in range(E):
        lo, hi = int(offs[e]), int(offs[e + 1])
        if hi > lo:
            ref = O.block_fp8_matmul_fp32(a[lo:hi], wq[e], sa[lo:hi], ws[e]).to(torch.bfloat16)
            assert O.rel_l2(out[lo:hi].float().cpu(), ref.float()) <= 1e-3, e


def test_fused_moe_small_vs_oracle_and_golden():
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8
    g = load_golden("moe_native.npz")
    a = as_bf16(g["a"])
    w1q, w2q, w1s, w2s = as_fp8(g["w1q"]), as_fp8(g["w2q"]), t(g["w1s"]), t(g["w2s"])
    score, topk = t(g["score"]), int(g["topk"])
    w, ids = O.fused_topk_native(score, topk)
    out = fused_experts_block_fp8(a.cuda(), w1q.cuda(), w2q.cuda(), w1s.cuda(), w2s.cuda(), w.cuda(), ids.cuda()).cpu()
    ref_seq = O.cutlass_fused_experts_fp8(a, w1q, w2q, w1s, w2s, w, ids)
    assert O.rel_l2(out.float(), ref_seq.float()) <= 5e-3        # same op order; silu uses __expf
    # the reference's own torch MoE (different bf16 rounding points): its tolerance is 2e-2 mean-rel-err
    assert O.mean_rel_err(out, as_bf16(g["out"])) < 2e-2
    _status_ok()


def test_fused_moe_deepseek_shapes_reduced_tokens():
    """E=32 local experts of the DeepSeek-V3 MoE (hidden 7168, intermediate 2048), 96 tokens, top-8."""
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8
    E, H, I, m, topk = 32, 7168, 2048, 96, 8
    g = torch.Generator().manual_seed(4)
    a = torch.randn(m, H, generator=g).to(torch.bfloat16)
    w13q, w13s, w2q, w2s = [], [], [], []
    for e in range(E):
        q_, s_ = O.per_block_cast_to_fp8(torch.randn(2 * I, H, generator=g) * 0.02); w13q.append(q_); w13s.append(s_)
        q_, s_ = O.per_block_cast_to_fp8(torch.randn(H, I, generator=g) * 0.02); w2q.append(q_); w2s.append(s_)
    w13q, w13s, w2q, w2s = torch.stack(w13q), torch.stack(w13s), torch.stack(w2q), torch.stack(w2s)
    w, ids = O.fused_topk_native(torch.randn(m, E, generator=g), topk)
    out = fused_experts_block_fp8(a.cuda(), w13q.cuda(), w2q.cuda(), w13s.cuda(), w2s.cuda(), w.cuda(), ids.cuda())
    out2 = fused_experts_block_fp8(a.cuda(), w13q.cuda(), w2q.cuda(), w13s.cuda(), w2s.cuda(), w.cuda(), ids.cuda())
    assert same_bits(out, out2)
    ref = O.cutlass_fused_experts_fp8(a, w13q, w2q, w13s, w2s, w, ids)
    assert O.rel_l2(out.float().cpu(), ref.float()) <= 5e-3
    _status_ok()


def _gpu_block_matmul_fp32(a_q, w_q, sa, sw):
    """fp32 restatement on the GPU of the block-scaled product (the arithmetic of native_w8a8_block_fp8_matmul,
    python/sglang/test/test_block_fp8.py:274-326): a_q [m,K] e4m3, w_q [N,K] e4m3, sa [m,K/128], sw [N/128,K/128]."""
    K = a_q.shape[1]
    c = torch.zeros(a_q.shape[0], w_q.shape[0], device=a_q.device)
    sw_rows = sw.repeat_interleave(128, 0)
    for kb in range(K // 128):
        c += (a_q[:, kb * 128:(kb + 1) * 128].float() @ w_q[:, kb * 128:(kb + 1) * 128].float().t()) * \
             (sa[:, kb:kb + 1] * sw_rows[:, kb][None, :])
    return c


def test_fused_moe_full_benchmark_size_256_experts_4096_tokens():
    """The MoE benchmark configuration at size on one GPU: 256 experts (hidden 7168, intermediate 2048, 11.3 GB of
    e4m3 weights), 4096 tokens, softmax top-8.  Every token against an fp32 restatement of the op sequence on the
    GPU (per expert: quantise, block-scaled product, bf16, SiLU*mul, quantise, product, bf16; weighted sum in fp32),
    and a sample of tokens against the CPU oracle run on just the experts those tokens use."""
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8
    old_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        E, H, I, m, topk = 256, 7168, 2048, 4096, 8
        dev = torch.device("cuda")
        w13 = torch.empty(E, 2 * I, H, dtype=torch.float8_e4m3fn, device=dev)
        w2 = torch.empty(E, H, I, dtype=torch.float8_e4m3fn, device=dev)
        w13s = torch.empty(E, 2 * I // 128, H // 128, device=dev)
        w2s = torch.empty(E, H // 128, I // 128, device=dev)
        g = torch.Generator(device=dev).manual_seed(40)

        def block_quant(w):   # per_block_cast_to_fp8 (sgl-kernel/tests/test_fp8_blockwise_moe.py:51-64) on the device
            n, k = w.shape
            wv = w.view(n // 128, 128, k // 128, 128)
            amax = wv.abs().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
            return (wv * (448.0 / amax)).to(torch.float8_e4m3fn).view(n, k), (amax / 448.0).view(n // 128, k // 128)
        for e in range(E):
            w13[e], w13s[e] = block_quant(torch.randn(2 * I, H, generator=g, device=dev) * 0.02)
            w2[e], w2s[e] = block_quant(torch.randn(H, I, generator=g, device=dev) * 0.02)
        x = torch.randn(m, H, generator=g, device=dev).to(torch.bfloat16)
        logits = torch.randn(m, E, generator=g, device=dev)
        tw, ti = torch.topk(torch.softmax(logits.float(), dim=-1), topk, dim=-1)
        ti = ti.to(torch.int32)
        out = fused_experts_block_fp8(x, w13, w2, w13s, w2s, tw, ti)
        out2 = fused_experts_block_fp8(x, w13, w2, w13s, w2s, tw, ti)
        assert same_bits(out, out2), "not deterministic"

        # fp32 restatement on the GPU, expert by expert
        def quant(t_):
            tf = t_.float().view(t_.shape[0], -1, 128)
            amax_ = tf.abs().amax(-1).clamp(min=1e-10)
            s_ = amax_ / torch.full_like(amax_, 448.0)   # tensor / tensor: an IEEE division on CUDA too
            return (tf / s_.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(t_.shape), s_
        xq, xs = quant(x)
        ref = torch.zeros(m, H, device=dev)
        flat_e = ti.reshape(-1).long()
        flat_t = torch.arange(m, device=dev).repeat_interleave(topk)
        flat_w = tw.to(torch.bfloat16).float().reshape(-1)
        contrib = torch.empty(m * topk, H, device=dev, dtype=torch.bfloat16)
        for e in range(E):
            sel = (flat_e == e).nonzero().flatten()
            if sel.numel() == 0:
                continue
            rows = flat_t[sel]
            c1 = _gpu_block_matmul_fp32(xq[rows], w13[e], xs[rows], w13s[e]).to(torch.bfloat16)
            act = (torch.nn.functional.silu(c1[:, :I].float()) * c1[:, I:].float()).to(torch.bfloat16)
            aq, as_ = quant(act)
            contrib[sel] = _gpu_block_matmul_fp32(aq, w2[e], as_, w2s[e]).to(torch.bfloat16)
        ref = (contrib.float().view(m, topk, H) * flat_w.view(m, topk, 1)).sum(1)
        err = O.rel_l2(out.float().cpu(), ref.to(torch.bfloat16).float().cpu())
        assert err <= 5e-3, err      # same tolerance as the small cases: __expf in SiLU, bf16 rounding flips
        # sampled tokens against the CPU oracle, restricted to the experts they route to
        tok = torch.arange(0, m, 683, device=dev)          # 6 tokens
        used = torch.unique(ti[tok].reshape(-1)).long()
        remap = torch.full((E,), -1, dtype=torch.int32, device=dev)
        remap[used] = torch.arange(used.numel(), dtype=torch.int32, device=dev)
        ids_local = remap[ti[tok].long()]
        ref_cpu = O.cutlass_fused_experts_fp8(x[tok].cpu(), w13[used].cpu(), w2[used].cpu(), w13s[used].cpu(),
                                              w2s[used].cpu(), tw[tok].cpu(), ids_local.cpu())
        assert O.rel_l2(out[tok].float().cpu(), ref_cpu.float()) <= 5e-3
        _status_ok()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old_tf32


def test_ep_module_single_rank_equals_fused_path():
    """world size 1: dispatch -> local grouped experts -> combine must give the fused path's bits."""
    from sglang_b200.distributed import ExpertParallelBlockFp8MoE
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8
    E, H, I, m, topk = 8, 512, 256, 70, 2
    g = torch.Generator().manual_seed(6)
    a = torch.randn(m, H, generator=g).to(torch.bfloat16).cuda()
    w13q, w13s, w2q, w2s = [], [], [], []
    for e in range(E):
        q_, s_ = O.per_block_cast_to_fp8(torch.randn(2 * I, H, generator=g) * 0.05); w13q.append(q_); w13s.append(s_)
        q_, s_ = O.per_block_cast_to_fp8(torch.randn(H, I, generator=g) * 0.05); w2q.append(q_); w2s.append(s_)
    w13q, w13s, w2q, w2s = [torch.stack(v).cuda() for v in (w13q, w13s, w2q, w2s)]
    w, ids = O.fused_topk_native(torch.randn(m, E, generator=g), topk)
    w, ids = w.cuda(), ids.cuda()
    ref = fused_experts_block_fp8(a, w13q, w2q, w13s, w2s, w, ids)
    moe = ExpertParallelBlockFp8MoE(w13q, w2q, w13s, w2s)
    out = moe(a, w, ids)
    assert same_bits(out, ref)
    _status_ok()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K", [(1, 128), (77, 2048), (300, 512)])
def test_fused_silu_mul_quant_equals_two_kernels(M, K, dtype):
    from sglang_b200.layers.quantization.fp8_kernel import (sglang_per_token_group_quant_fp8,
                                                            silu_and_mul_per_token_group_quant_fp8)
    from sglang_b200.sgl_kernel import silu_and_mul
    g = torch.Generator().manual_seed(M + K)
    x = (torch.randn(M, 2 * K, generator=g) * 2).to(dtype).cuda()
    q_ref, s_ref = sglang_per_token_group_quant_fp8(silu_and_mul(x), 128)
    q, s = silu_and_mul_per_token_group_quant_fp8(x, 128)
    assert same_bits(q, q_ref) and same_bits(s, s_ref)
    q2, s2 = silu_and_mul_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True)
    assert same_bits(q2, q_ref) and same_bits(s2.contiguous(), s_ref)
    # and directly against the CPU oracle: SiLU*mul in fp32 rounded once to the input type, then the group quantiser.
    # The kernel evaluates the exponential with __expf, so a rounded activation may differ by one ulp of the input
    # type now and then; codes may then differ by one step in that group.  Scales within 1 ulp-of-input relative,
    # dequantised values within one e4m3 step of the oracle's.
    xc = x.cpu()
    act = O.silu_and_mul(xc)
    qo, so = O.quant_group_fp8_cuda_semantics(act, 128)
    rel = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10}[dtype]
    assert torch.allclose(s.cpu(), so, rtol=2 * rel, atol=0)
    deq, deq_o = q.float().cpu().view(M, -1, 128) * s.cpu().unsqueeze(-1), qo.float().view(M, -1, 128) * so.unsqueeze(-1)
    assert bool(((deq - deq_o).abs() <= so.unsqueeze(-1) * 32.0 + 1e-30).all())
    assert (q.cpu().view(torch.uint8) != qo.view(torch.uint8)).float().mean() < 0.05


def test_fp8_moe_method_apply():
    """Fp8MoEMethod owning the expert weights ([E, 2I, H] / [E, H, I]): create -> load -> apply, equal to the
    fused path called directly and within tolerance of the oracle; routed_scaling_factor is applied last."""
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8
    from sglang_b200.layers.quantization.fp8 import Fp8Config, Fp8MoEMethod
    E, H, I, m, topk = 8, 512, 256, 64, 2
    g = torch.Generator().manual_seed(9)
    method = Fp8MoEMethod(Fp8Config.from_config(
        {"quant_method": "fp8", "activation_scheme": "dynamic", "weight_block_size": [128, 128]}))
    layer = torch.nn.Module()
    method.create_weights(layer, E, H, I, torch.bfloat16, device="cuda")
    w13q, w13s, w2q, w2s = [], [], [], []
    for e in range(E):
        q_, s_ = O.per_block_cast_to_fp8(torch.randn(2 * I, H, generator=g) * 0.05); w13q.append(q_); w13s.append(s_)
        q_, s_ = O.per_block_cast_to_fp8(torch.randn(H, I, generator=g) * 0.05); w2q.append(q_); w2s.append(s_)
    w13q, w13s, w2q, w2s = torch.stack(w13q), torch.stack(w13s), torch.stack(w2q), torch.stack(w2s)
    layer.w13_weight.data.copy_(w13q.cuda()); layer.w2_weight.data.copy_(w2q.cuda())
    layer.w13_weight_scale_inv.data.copy_(w13s.cuda()); layer.w2_weight_scale_inv.data.copy_(w2s.cuda())
    a = torch.randn(m, H, generator=g).to(torch.bfloat16)
    w, ids = O.fused_topk_native(torch.randn(m, E, generator=g), topk)
    out = method.apply(layer, a.cuda(), (w.cuda(), ids.cuda(), None))
    direct = fused_experts_block_fp8(a.cuda(), w13q.cuda(), w2q.cuda(), w13s.cuda(), w2s.cuda(), w.cuda(), ids.cuda())
    assert same_bits(out, direct)
    ref = O.cutlass_fused_experts_fp8(a, w13q, w2q, w13s, w2s, w, ids)
    assert O.rel_l2(out.float().cpu(), ref.float()) <= 5e-3
    scaled = method.apply(layer, a.cuda(), (w.cuda(), ids.cuda(), None), routed_scaling_factor=2.5)
    assert same_bits(scaled, direct * 2.5)
    _status_ok()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,E,topk", [(1, 8, 2), (37, 64, 6), (513, 256, 8), (100, 160, 6), (9, 1024, 32), (33, 4, 4)])
@pytest.mark.parametrize("renorm", [False, True])
def test_topk_softmax_router(m, E, topk, dtype, renorm):
    """softmax(logits.float()) -> top-k against the torch form (python/sglang/srt/layers/moe/topk.py:284-302):
    weights to 1e-6 relative, ids exact wherever the k-th and (k+1)-th probabilities are not within rounding."""
    from sglang_b200.layers.moe.topk import fused_topk
    g = torch.Generator().manual_seed(m * 7 + E + topk)
    logits = (torch.randn(m, E, generator=g) * 3).to(dtype)
    w, ids = fused_topk(torch.empty(m, 1, device="cuda"), logits.cuda(), topk, renorm)
    assert w.dtype == torch.float32 and ids.dtype == torch.int32 and w.shape == (m, topk)
    probs = torch.softmax(logits.float(), dim=-1)
    w_ref, ids_ref = torch.topk(probs, topk, dim=-1)
    if renorm:
        w_ref = w_ref / w_ref.sum(dim=-1, keepdim=True)
    torch.testing.assert_close(w.cpu(), w_ref, rtol=2e-6, atol=1e-9)
    # the picked experts carry the picked probabilities; exact id equality except at rounding-level ties
    picked = probs.gather(1, ids.cpu().long())
    if renorm:
        picked = picked / picked.sum(dim=-1, keepdim=True)
    torch.testing.assert_close(picked, w_ref, rtol=2e-6, atol=1e-9)
    srt = torch.sort(probs, dim=-1, descending=True).values
    clear = (srt[:, :-1] - srt[:, 1:]).abs().min(dim=-1).values > 1e-7 if E > 1 else torch.ones(m, dtype=torch.bool)
    assert torch.equal(ids.cpu()[clear], ids_ref.to(torch.int32)[clear])
    assert bool((ids.cpu().sort(dim=-1).values.diff(dim=-1) != 0).all()) if topk > 1 else True


def test_topk_softmax_ties_and_moe_pipeline():
    """Equal logits: the lower expert ids win, in order.  Then router -> fused experts on the device, equal to the
    same call fed with the oracle's routing."""
    from sglang_b200.layers.moe.topk import fused_topk
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8
    flat = torch.zeros(3, 16, device="cuda")
    w, ids = fused_topk(flat, flat, 4, False)
    assert torch.equal(ids.cpu(), torch.arange(4, dtype=torch.int32).repeat(3, 1))
    torch.testing.assert_close(w.cpu(), torch.full((3, 4), 1 / 16))
    g = torch.Generator().manual_seed(3)
    E, H, I, m, topk = 8, 256, 128, 40, 2
    w13q, w13s, w2q, w2s = [], [], [], []
    for _ in range(E):
        q_, s_ = O.per_block_cast_to_fp8(torch.randn(2 * I, H, generator=g) * 0.05); w13q.append(q_); w13s.append(s_)
        q_, s_ = O.per_block_cast_to_fp8(torch.randn(H, I, generator=g) * 0.05); w2q.append(q_); w2s.append(s_)
    w13q, w13s, w2q, w2s = (torch.stack(v).cuda() for v in (w13q, w13s, w2q, w2s))
    a = torch.randn(m, H, generator=g).to(torch.bfloat16).cuda()
    score = torch.randn(m, E, generator=g)
    tw, ti = fused_topk(a, score.cuda(), topk, False)
    tw_ref, ti_ref = O.fused_topk_native(score, topk)
    assert torch.equal(ti.cpu(), ti_ref)
    out = fused_experts_block_fp8(a, w13q, w2q, w13s, w2s, tw, ti)
    out_ref = fused_experts_block_fp8(a, w13q, w2q, w13s, w2s, tw_ref.cuda(), ti_ref.cuda())
    assert O.rel_l2(out.float().cpu(), out_ref.float().cpu()) <= 1e-3
    _status_ok()


def _biased_grouped_topk_ref(logits, bias, G, topk_group, topk):
    """The torch form of python/sglang/srt/layers/moe/topk.py:477-524 (renormalize=True, no shared experts)."""
    scores = logits.sigmoid()
    m, E = scores.shape
    choice = scores + bias.unsqueeze(0)
    group_scores = choice.view(m, G, -1).topk(2, dim=-1)[0].sum(dim=-1)
    group_idx = torch.topk(group_scores, k=topk_group, dim=-1, sorted=False)[1]
    group_mask = torch.zeros_like(group_scores).scatter_(1, group_idx, 1)
    score_mask = group_mask.unsqueeze(-1).expand(m, G, E // G).reshape(m, -1)
    tmp = choice.masked_fill(~score_mask.bool(), float("-inf"))
    _, ids = torch.topk(tmp, k=topk, dim=-1)
    w = scores.gather(1, ids)
    return w / w.sum(dim=-1, keepdim=True), ids


@pytest.mark.parametrize("m,E,G,topk_group,topk", [(1, 256, 8, 4, 8), (300, 256, 8, 4, 8), (77, 64, 4, 2, 6),
                                                   (40, 512, 16, 4, 8), (5, 16, 8, 8, 16), (64, 128, 32, 3, 5)])
def test_moe_fused_gate(m, E, G, topk_group, topk):
    from sglang_b200.sgl_kernel import moe_fused_gate
    g = torch.Generator().manual_seed(m + E + G)
    logits = torch.randn(m, E, generator=g) * 2
    bias = torch.randn(E, generator=g) * 0.1
    w, ids = moe_fused_gate(logits.cuda(), bias.cuda(), G, topk_group, topk)
    w_ref, ids_ref = _biased_grouped_topk_ref(logits, bias, G, topk_group, topk)
    # same SET of experts per token (the reference does not order them), same weights per expert
    got = torch.zeros(m, E).scatter_(1, ids.cpu().long(), w.cpu())
    want = torch.zeros(m, E).scatter_(1, ids_ref, w_ref)
    assert torch.equal(got != 0, want != 0)
    torch.testing.assert_close(got, want, rtol=3e-6, atol=1e-8)
    torch.testing.assert_close(w.sum(dim=-1).cpu(), torch.ones(m), rtol=1e-5, atol=1e-6)
    # fused shared experts (sgl-kernel/csrc/moe/moe_fused_gate.cu:225-252): the last n slots carry ids E, E+1, ... and
    # weight 1 / routed_scaling_factor; the routed slots before them are the gate with topk - n choices
    for n_shared in (1, 2):
        if topk - n_shared < 1:
            continue
        w2, ids2 = moe_fused_gate(logits.cuda(), bias.cuda(), G, topk_group, topk, num_fused_shared_experts=n_shared,
                                  routed_scaling_factor=2.5)
        w_r, ids_r = moe_fused_gate(logits.cuda(), bias.cuda(), G, topk_group, topk - n_shared)
        assert torch.equal(ids2[:, :topk - n_shared], ids_r) and torch.equal(w2[:, :topk - n_shared], w_r)
        assert torch.equal(ids2[:, topk - n_shared:].cpu(),
                           (E + torch.arange(n_shared, dtype=torch.int32)).repeat(m, 1))
        torch.testing.assert_close(w2[:, topk - n_shared:].cpu(), torch.full((m, n_shared), 1 / 2.5), rtol=1e-6, atol=0)
    # the operator registered with the reference's schema returns the same pair
    w3, ids3 = torch.ops.sgl_kernel.moe_fused_gate(logits.cuda(), bias.cuda(), G, topk_group, topk, 0, 1.0)
    assert torch.equal(w3, w) and torch.equal(ids3, ids)


def test_checkpoint_to_moe_layer(tmp_path):
    """A synthetic safetensors checkpoint (Hugging Face naming) -> Fp8MoEMethod parameters on the device for one
    expert-parallel rank's experts -> router -> fused experts, against the oracle on the same tensors."""
    import json
    from safetensors.torch import save_file
    from sglang_b200.layers.moe.topk import fused_topk
    from sglang_b200.layers.quantization.fp8 import Fp8MoEMethod
    from sglang_b200.model_loader.block_fp8_checkpoint import (SafetensorsIndex, expert_range, load_experts,
                                                               read_quantization_config)
    E, H, I, m, topk = 4, 256, 128, 32, 2
    g = torch.Generator().manual_seed(21)
    tensors, w13q, w13s, w2q, w2s = {}, [], [], [], []
    for e in range(E):
        gq, gs = O.per_block_cast_to_fp8(torch.randn(I, H, generator=g) * 0.05)
        uq, us = O.per_block_cast_to_fp8(torch.randn(I, H, generator=g) * 0.05)
        dq, ds = O.per_block_cast_to_fp8(torch.randn(H, I, generator=g) * 0.05)
        p = f"model.layers.3.mlp.experts.{e}."
        tensors.update({p + "gate_proj.weight": gq, p + "gate_proj.weight_scale_inv": gs.contiguous(),
                        p + "up_proj.weight": uq, p + "up_proj.weight_scale_inv": us.contiguous(),
                        p + "down_proj.weight": dq, p + "down_proj.weight_scale_inv": ds.contiguous()})
        w13q.append(torch.cat([gq, uq])); w13s.append(torch.cat([gs, us])); w2q.append(dq); w2s.append(ds)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({"quantization_config": {
        "quant_method": "fp8", "activation_scheme": "dynamic", "weight_block_size": [128, 128]}}))
    method = Fp8MoEMethod(read_quantization_config(str(tmp_path)))
    layer = torch.nn.Module()
    method.create_weights(layer, E, H, I, torch.bfloat16, device="cuda")
    load_experts(method, layer, SafetensorsIndex(str(tmp_path)), "model.layers.3.mlp.experts", expert_range(E, 0, 1))
    a = torch.randn(m, H, generator=g).to(torch.bfloat16)
    score = torch.randn(m, E, generator=g)
    tw, ti = fused_topk(a.cuda(), score.cuda(), topk, False)
    out = method.apply(layer, a.cuda(), (tw, ti, None)).cpu()
    tw_ref, ti_ref = O.fused_topk_native(score, topk)
    ref = O.cutlass_fused_experts_fp8(a, torch.stack(w13q), torch.stack(w2q), torch.stack(w13s), torch.stack(w2s),
                                      tw_ref, ti_ref)
    assert O.rel_l2(out.float(), ref.float()) <= 5e-3
    _status_ok()


@pytest.mark.parametrize("pad", [True, False])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("block_size,m,topk,E", [
    (4, 4, 3, 4), (32, 1, 1, 64), (64, 16, 8, 256), (128, 128, 8, 256), (32, 512, 8, 257), (128, 511, 8, 256),
    (256, 513, 8, 160), (16, 4096, 8, 256), (128, 4099, 6, 260), (64, 2048, 2, 8), (128, 16384, 8, 256)])
def test_moe_align_block_size_exact(block_size, m, topk, E, dtype, pad):
    """Shapes of sgl-kernel/tests/test_moe_align.py:140-151 (block sizes, token counts, expert counts incl. the
    non-power-of-two ones) through the reference's call convention (num_experts + 1 slots, caller-sized buffers,
    fused_moe.py:598-627).  Everything the op defines is compared exactly: padded length, the block -> expert
    table, the prefix, and sorted_token_ids (ascending inside an expert, `numel` in the padding)."""
    from sglang_b200.sgl_kernel import moe_align_block_size
    g = torch.Generator().manual_seed(block_size + m + E)
    ids = torch.argsort(torch.rand(m, E, generator=g), dim=1)[:, :topk].to(dtype)
    if m >= 16:
        ids[3, 0] = -1                                   # an expert filtered out by expert parallelism
        ids[m - 1, topk - 1] = -1
    numel = ids.numel()
    cap = numel + (E + 1) * (block_size - 1)
    sorted_ids = torch.empty(cap, dtype=torch.int32, device="cuda")
    if not pad:
        sorted_ids.fill_(numel)
    nblocks = (cap + block_size - 1) // block_size
    expert_ids = torch.zeros(nblocks, dtype=torch.int32, device="cuda")
    post = torch.empty(1, dtype=torch.int32, device="cuda")
    cumsum = torch.empty(E + 2, dtype=torch.int32, device="cuda")
    torch.ops.sgl_kernel.moe_align_block_size(ids.cuda(), E + 1, block_size, sorted_ids, expert_ids, post, cumsum, pad)
    s_ref, e_ref, total, c_ref = O.moe_align_block_size(ids, E + 1, block_size, cap)
    assert int(post.item()) == total
    assert torch.equal(cumsum.cpu()[: E + 2], c_ref)
    assert torch.equal(expert_ids.cpu()[: total // block_size], e_ref[: total // block_size])
    assert torch.equal(sorted_ids.cpu()[:total], s_ref[:total])
    if not pad:
        assert bool((sorted_ids.cpu()[total:] == numel).all())     # nothing written past the padded length
    # size-independent properties: a permutation of the valid flat indices, each in a block of its own expert
    got = sorted_ids.cpu()[:total].long()
    real = got[got < numel]
    flat = ids.reshape(-1).long()
    assert torch.equal(real.sort().values, torch.nonzero(flat >= -1).squeeze(1))
    pos = torch.nonzero(got < numel).squeeze(1)
    assert torch.equal(expert_ids.cpu().long()[pos // block_size], flat[real])


def test_moe_align_block_size_docstring_example_and_errors():
    """The worked example of fused_moe.py:583-596 (ids shifted to start at 0), and the argument checks."""
    from sglang_b200.sgl_kernel import moe_align_block_size
    ids = (torch.tensor([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]], dtype=torch.int32) - 1).cuda()
    sorted_ids = torch.empty(12 + 5 * 3, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(7, dtype=torch.int32, device="cuda")
    post = torch.empty(1, dtype=torch.int32, device="cuda")
    cumsum = torch.empty(6, dtype=torch.int32, device="cuda")
    moe_align_block_size(ids, 5, 4, sorted_ids, expert_ids, post, cumsum, True)
    assert int(post.item()) == 16
    assert sorted_ids.cpu()[:16].tolist() == [3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12]
    assert expert_ids.cpu()[:4].tolist() == [0, 1, 2, 3]
    with pytest.raises(RuntimeError):
        moe_align_block_size(ids.float(), 5, 4, sorted_ids, expert_ids, post, cumsum, True)
    with pytest.raises(RuntimeError):
        moe_align_block_size(ids, 5, 4, sorted_ids, expert_ids, post, cumsum[:3], True)

"""CPU: pin the oracle against vectors produced by the reference's own functions
(tests/golden/make_golden.py) and its known-answer generators."""
import numpy as np
import torch

from oracle import block_fp8_oracle as O
from helpers import as_bf16, as_f16, as_fp8, load_golden, same_bits, t


def test_quant_matches_reference_torch_twin():
    g = load_golden("quant_native.npz")
    for name, conv in (("bf16", as_bf16), ("f16", as_f16), ("f32", t)):
        x = conv(g[f"rand_{name}_x"])
        for fn in (O.native_per_token_group_quant_fp8, O.quant_group_fp8_cuda_semantics):
            q, s = fn(x, 128)
            assert same_bits(q, as_fp8(g[f"rand_{name}_q"])), (name, fn.__name__)
            assert same_bits(s, t(g[f"rand_{name}_s"])), (name, fn.__name__)
    x = as_bf16(g["randn_bf16_x"])
    for fn in (O.native_per_token_group_quant_fp8, O.quant_group_fp8_cuda_semantics):
        q, s = fn(x, 128)
        assert same_bits(q, as_fp8(g["randn_bf16_q"]))
        assert same_bits(s, t(g["randn_bf16_s"]))


def test_quant_ue8m0_matches_reference_functions():
    """Power-of-two scales: the reference's torch functions (make_golden.py --only ue8m0) vs the oracle's
    restatements, and the CUDA-semantics form (eps 1e-10, division) on the same non-degenerate inputs."""
    g = load_golden("quant_ue8m0.npz")
    for xk, qk, sk, conv in (("x", "xq", "xs", as_bf16), ("x32", "x32q", "x32s", t)):
        x = conv(g[xk])
        q, s = O.per_token_group_quant_mxfp8(x)
        assert same_bits(q, as_fp8(g[qk])) and same_bits(s, t(g[sk]))
        q2, s2, packed = O.quant_group_fp8_ue8m0_cuda_semantics(x, 128)
        assert same_bits(q2, as_fp8(g[qk])) and same_bits(s2, t(g[sk]))
        # the packed bytes decode to the same powers of two
        G = s2.shape[1]
        by = torch.stack([(packed >> (8 * b)) & 0xFF for b in range(4)], dim=-1).reshape(s2.shape[0], -1)
        assert torch.equal(torch.pow(2.0, (by[:, :G] - 127).float()), s2)
        assert bool((by[:, G:] == 0).all())
    wq, ws = O.per_block_quant_mxfp8(t(g["w"]))
    assert same_bits(wq, as_fp8(g["wq"])) and same_bits(ws, t(g["ws"]))


def test_rmsnorm_matches_reference_forward_native():
    """RMSNorm.forward_native executed by make_golden.py --only rmsnorm vs the oracle's restatement: same bits."""
    g = load_golden("rmsnorm_native.npz")
    for name, conv in (("bf16", as_bf16), ("f16", as_f16)):
        x, r, w = conv(g[f"{name}_x"]), conv(g[f"{name}_r"]), conv(g[f"{name}_w"])
        assert same_bits(O.rmsnorm_native(x, w, 1e-6), conv(g[f"{name}_y"]))
        y2, r2 = O.rmsnorm_native(x, w, 1e-6, r)
        assert same_bits(y2, conv(g[f"{name}_y_res"])) and same_bits(r2, conv(g[f"{name}_r_out"]))


def test_int8_quant_matches_reference_native():
    """native_per_token_group_quant_int8 (test/srt/quant/test_block_int8.py:13-35) executed by
    make_golden.py --only int8 vs the oracle's restatement of the CUDA kernel's int8 destination: same codes, same
    scales (no all-zero group in these inputs, the one case where the torch twin clamps eps in the input type)."""
    g = load_golden("quant_int8_native.npz")
    for name, conv in (("bf16", as_bf16), ("f16", as_f16), ("f32", t)):
        x = conv(g[f"{name}_x"])
        for group in (64, 128):
            q, s = O.quant_group_int8_cuda_semantics(x, group)
            assert torch.equal(q, torch.from_numpy(g[f"{name}_g{group}_q"]))
            assert same_bits(s, t(g[f"{name}_g{group}_s"]).reshape(s.shape))


def test_quant_known_answer():
    """test/srt/quant/test_fp8_kernel.py:90-100: scales equal, <1e-4 of codes differ."""
    g = load_golden("known_answer.npz")
    A, A_q, A_s = t(g["A"]), as_fp8(g["A_q"]), t(g["A_s"])
    q, s = O.quant_group_fp8_cuda_semantics(A, 128)
    torch.testing.assert_close(s, A_s)
    diff = (q.to(torch.float16) - A_q.to(torch.float16)).abs()
    assert (diff > 1e-5).count_nonzero() / diff.numel() < 1e-4


def test_matmul_matches_reference_native():
    g = load_golden("matmul_native.npz")
    a, b, As, Bs = as_fp8(g["a"]), as_fp8(g["b"]), t(g["As"]), t(g["Bs"])
    c = O.block_fp8_matmul_fp32(a, b, As, Bs)
    ref = t(g["c_f32"])
    assert O.rel_l2(c, ref) < 1e-6
    cb = O.native_w8a8_block_fp8_matmul(a, b, As, Bs, [128, 128], torch.bfloat16)
    assert O.rel_l2(cb.float(), as_bf16(g["c_bf16"]).float()) < 1e-4
    base = O.baseline_scaled_mm(a, b.t(), As, Bs.t(), torch.bfloat16)
    assert O.rel_l2(base.float(), as_bf16(g["baseline_bf16"]).float()) < 1e-4
    # the two reference formulations agree with each other to bf16 noise
    assert O.rel_l2(cb.float(), base.float()) < 3e-3


def test_matmul_known_answer():
    """test/srt/quant/test_fp8_kernel.py:103-122: atol 0.5, rtol 1e-4 vs bf16 product."""
    g = load_golden("known_answer.npz")
    A, A_q, A_s = t(g["A"]), as_fp8(g["A_q"]), t(g["A_s"])
    B, B_q, B_s = t(g["B"]), as_fp8(g["B_q"]), t(g["B_s"])
    C_gt = A.to(torch.bfloat16) @ B.to(torch.bfloat16)
    C = O.native_w8a8_block_fp8_matmul(A_q, B_q.T.contiguous(), A_s, B_s.T.contiguous(), [128, 128], torch.bfloat16)
    torch.testing.assert_close(C, C_gt, atol=0.5, rtol=1e-4)


def test_casts():
    g = load_golden("casts.npz")
    wq, ws = O.per_block_cast_to_fp8(t(g["w"]))
    assert same_bits(wq, as_fp8(g["wq"])) and same_bits(ws, t(g["ws"]))
    tq, ts = O.per_token_cast_to_fp8(t(g["t"]))
    assert same_bits(tq.contiguous(), as_fp8(g["tq"])) and same_bits(ts, t(g["ts"]))
    d = O.calc_diff(torch.randn(64, 64, generator=torch.Generator().manual_seed(3)),
                    torch.randn(64, 64, generator=torch.Generator().manual_seed(4)))
    assert abs(d - float(g["calc_diff"])) < 1e-12


def test_moe_matches_reference_native():
    g = load_golden("moe_native.npz")
    a = as_bf16(g["a"])
    w1q, w2q, w1s, w2s = as_fp8(g["w1q"]), as_fp8(g["w2q"]), t(g["w1s"]), t(g["w2s"])
    score, topk = t(g["score"]), int(g["topk"])
    ref = as_bf16(g["out"]).float()
    o = O.torch_w8a8_block_fp8_moe(a, w1q, w2q, w1s, w2s, score, topk).float()
    assert O.rel_l2(o, ref) < 1e-6
    # op-sequence oracle (cutlass_moe.py order: quantise once, gather codes; fp32 silu*mul and
    # fp32 weighted sum, each rounded once) differs from the torch twin only by where bf16
    # rounding happens; the reference's own MoE tolerance is 2e-2 (test_block_fp8.py:521-525)
    w, ids = O.fused_topk_native(score, topk)
    o2 = O.cutlass_fused_experts_fp8(a, w1q, w2q, w1s, w2s, w, ids).float()
    assert O.rel_l2(o2, ref) < 3e-2


def test_prepare_moe_input_properties():
    torch.manual_seed(0)
    ids = torch.randint(0, 8, (37, 2), dtype=torch.int32)
    offs, ps1, ps2, a_map, c_map = O.prepare_moe_input(ids, 8, 64, 256)
    assert offs[0] == 0 and offs[-1] == ids.numel()
    flat = ids.reshape(-1)
    for e in range(8):
        assert int(ps1[e, 0]) == int((flat == e).sum()) and tuple(ps1[e, 1:].tolist()) == (128, 256)
        assert tuple(ps2[e].tolist()) == (int((flat == e).sum()), 256, 64)
    # slot s holds token a_map[s]; c_map inverts it
    for i in range(flat.numel()):
        s = int(c_map[i]); e = int(flat[i])
        assert int(offs[e]) <= s < int(offs[e + 1]) and int(a_map[s]) == i // 2


def test_zero_group_and_nan_follow_cuda_kernel():
    x = torch.zeros(2, 256, dtype=torch.bfloat16)
    x[1, 5] = float("nan"); x[1, 7] = 3.0
    q, s = O.quant_group_fp8_cuda_semantics(x, 128)
    assert float(s[0, 0]) == np.float32(1e-10) / np.float32(448.0)
    assert float(s[1, 0]) == np.float32(3.0) / np.float32(448.0)
    assert float(q[1, 5].float()) == -448.0 and float(q[1, 7].float()) == 448.0


def test_moe_align_block_size_docstring_example():
    """The oracle's moe_align_block_size against the worked example the reference gives for the op
    (python/sglang/srt/layers/moe/fused_moe_triton/fused_moe.py:583-596; its 1-based ids shifted to start at 0),
    plus the invariants of sgl-kernel/tests/test_moe_align.py on a random case with filtered (-1) ids."""
    ids = torch.tensor([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]]) - 1
    s, e, total, c = O.moe_align_block_size(ids, 5, 4)
    assert total == 16
    assert s[:16].tolist() == [3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12]
    assert e[:4].tolist() == [0, 1, 2, 3] and c.tolist() == [0, 0, 4, 8, 12, 16]
    g = torch.Generator().manual_seed(5)
    E, bs = 37, 16
    ids = torch.argsort(torch.rand(300, E, generator=g), dim=1)[:, :6]
    ids[7, 2] = -1
    s, e, total, c = O.moe_align_block_size(ids, E + 1, bs)
    flat = ids.reshape(-1)
    assert total % bs == 0 and int(c[-1]) == total and int(c[1]) == bs      # the single -1 pads to one block
    got = s[:total].long()
    real = got[got < flat.numel()]
    assert torch.equal(real.sort().values, torch.arange(flat.numel()))
    pos = torch.nonzero(got < flat.numel()).squeeze(1)
    assert torch.equal(e.long()[pos // bs], flat[real])
    assert bool((s[total:] == flat.numel()).all())

"""GPU parity: per-token-group FP8 quantisation, bit-exact against the CPU oracle.

Cases follow the reference's own tests (python/sglang/test/test_block_fp8.py:51-90,
sgl-kernel/tests/test_per_token_group_quant_8bit.py:220-316) and the benchmark's
quantisation configuration (N(0,1) with 0.1 % of entries x100, K = 7168).
"""
import numpy as np
import pytest
import torch

from oracle import block_fp8_oracle as O
from helpers import as_bf16, as_fp8, count_diff_bits, load_golden, same_bits, t

pytestmark = pytest.mark.gpu

LAYOUTS = [
    dict(column_major_scales=False, scale_tma_aligned=False),
    dict(column_major_scales=True, scale_tma_aligned=False),
    dict(column_major_scales=True, scale_tma_aligned=True),
]


def _quant(x, group=128, **kw):
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    return sglang_per_token_group_quant_fp8(x.cuda(), group, **kw)


def _check_exact(x, group=128, **kw):
    q, s = _quant(x, group, **kw)
    q_ref, s_ref = O.quant_group_fp8_cuda_semantics(x, group)
    assert s.shape == s_ref.shape
    nd_q = count_diff_bits(q.cpu(), q_ref)
    nd_s = count_diff_bits(s.cpu().contiguous(), s_ref)
    assert nd_q == 0 and nd_s == 0, f"{nd_q} codes / {nd_s} scales differ of {q_ref.numel()} / {s_ref.numel()}"
    return q, s


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("M", [1, 3, 7, 127, 128, 129, 2048])
def test_config2_distribution_bit_exact(M, layout):
    x = O.gen_activation(M, 7168, seed=2000 + M, outlier_frac=1e-3)
    q, s = _check_exact(x, **layout)
    if layout["column_major_scales"]:
        assert s.stride(0) == 1
        if layout["scale_tma_aligned"]:
            assert s.stride(1) == (M + 3) // 4 * 4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("group", [64, 128, 256, 512])
@pytest.mark.parametrize("shape", [(7, 512), (83, 4096), (33, 5120), (5, 13824)])
def test_reference_test_grid(shape, group, dtype):
    """Shapes/dtypes/groups of test_block_fp8.py:51-56 (torch.rand inputs, seed 0)."""
    torch.manual_seed(0)
    x = torch.rand(*shape, dtype=dtype)
    _check_exact(x, group)


def test_golden_vectors_and_known_answer():
    g = load_golden("quant_native.npz")
    x = as_bf16(g["randn_bf16_x"])
    q, s = _quant(x)
    assert same_bits(q.cpu(), as_fp8(g["randn_bf16_q"])) and same_bits(s.cpu(), t(g["randn_bf16_s"]))
    k = load_golden("known_answer.npz")
    q, s = _quant(t(k["A"]))
    torch.testing.assert_close(s.cpu(), t(k["A_s"]))
    diff = (q.cpu().to(torch.float16) - as_fp8(k["A_q"]).to(torch.float16)).abs()
    assert (diff > 1e-5).count_nonzero() / diff.numel() < 1e-4


def test_special_values():
    x = torch.zeros(8, 256, dtype=torch.bfloat16)
    x[1, 5] = float("nan"); x[1, 7] = 3.0
    x[2, 0] = float("inf"); x[2, 1] = 1.0
    x[3, :128] = 1e-30
    x[4, 3] = -65280.0; x[4, 4] = 2.0 ** -120
    x[5, 130] = -0.0
    x[6, :] = torch.finfo(torch.bfloat16).max
    _check_exact(x)
    xf = x.float()
    xf[7, 0] = 1.17549435e-38; xf[7, 1] = 3.4e38
    _check_exact(xf)


def test_fast_division_equals_ieee_division():
    """Both C-ABI entry points must produce identical bits on wide-ranging inputs,
    including scales whose significand is all ones."""
    from sglang_b200 import _lib
    g = torch.Generator().manual_seed(7)
    M, K = 4096, 2048
    x = torch.randn(M, K, generator=g) * torch.exp(torch.randn(M, 1, generator=g) * 8.0)
    # force all-ones-significand scales in some groups: amax = 448 * (2 - 2^-23) * 2^e
    amax = np.float32(448.0) * np.frombuffer(np.uint32(0x3fffffff).tobytes(), dtype=np.float32)[0]
    x[:64, 0] = float(amax)
    x[:64, 1:128] = x[:64, 1:128].clamp(-1.0, 1.0)
    for dt in (torch.float32, torch.bfloat16):
        xd = x.to(dt).cuda()
        outs = []
        for fn in ("b200_per_token_group_quant_fp8", "b200_per_token_group_quant_fp8_ieee_div"):
            q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
            s = torch.empty(M, K // 128, dtype=torch.float32, device="cuda")
            rc = getattr(_lib.lib(), fn)(xd.data_ptr(), {torch.float32: 0, torch.bfloat16: 2}[dt], q.data_ptr(),
                                         s.data_ptr(), M, K, 128, K // 128, 1, 1e-10, -448.0, 448.0,
                                         torch.cuda.current_stream().cuda_stream)
            _lib.check(fn, rc)
            outs.append((q, s))
        torch.cuda.synchronize()
        assert same_bits(outs[0][0], outs[1][0]) and same_bits(outs[0][1], outs[1][1])
        q_ref, s_ref = O.quant_group_fp8_cuda_semantics(x.to(dt), 128)
        assert same_bits(outs[0][0].cpu(), q_ref) and same_bits(outs[0][1].cpu(), s_ref)


def test_padding_rows_untouched_and_empty():
    from sglang_b200.sgl_kernel import sgl_per_token_group_quant_fp8
    M, K = 5, 256
    x = O.gen_activation(M, K, seed=11).cuda()
    q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
    buf = torch.full((K // 128, 8), 123.0, dtype=torch.float32, device="cuda")
    s = buf.t()[:M]
    sgl_per_token_group_quant_fp8(x, q, s, 128, 1e-10, -448.0, 448.0, False)
    assert torch.all(buf[:, M:] == 123.0)
    _, s_ref = O.quant_group_fp8_cuda_semantics(x.cpu(), 128)
    assert same_bits(s.contiguous().cpu(), s_ref)
    # M == 0: no launch, empty outputs
    q0, s0 = _quant(torch.empty(0, 256, dtype=torch.bfloat16))
    assert q0.shape == (0, 256) and s0.shape == (0, 2)


def test_full_size_checksum_property():
    """M = 16384 x 7168 (the bandwidth configuration): every row block must match the
    oracle; checked on strided row samples plus a dequantisation bound on everything."""
    M, K = 16384, 7168
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32)
    x = torch.where(torch.rand(M, K, generator=g, device="cuda") < 1e-3, x * 100, x).to(torch.bfloat16)
    q, s = _quant(x, column_major_scales=True, scale_tma_aligned=True)
    rows = torch.arange(0, M, 61)
    q_ref, s_ref = O.quant_group_fp8_cuda_semantics(x[rows.cuda()].cpu(), 128)
    assert same_bits(q[rows.cuda()].cpu(), q_ref) and same_bits(s[rows.cuda()].contiguous().cpu(), s_ref)
    # size-independent property: |dequant - x| <= scale * 2^-4 * 448 / 2 ... i.e. half an e4m3 ulp at amax
    deq = q.float().view(M, K // 128, 128) * s.unsqueeze(-1)
    err = (deq - x.float().view(M, K // 128, 128)).abs().amax(-1)
    assert bool(torch.all(err <= s * 16.001 + 1e-30))   # 16 = half the e4m3 step at the top binade


def test_largest_benchmark_size_m65536_every_element():
    """M = 65536 x 7168 (the largest size of the bandwidth configuration, 470 M elements): the CPU oracle on
    every 509th row, and EVERY code and scale bit for bit against a torch restatement of the same arithmetic on
    the GPU (fp32 divide, clamp, round-to-nearest-even saturating cast; itself pinned to the oracle on the
    sampled rows), row-major and column-major padded scale layouts."""
    M, K = 65536, 7168
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
    for r0 in range(0, M, 8192):
        blk = torch.randn(8192, K, generator=g, device="cuda", dtype=torch.float32)
        blk = torch.where(torch.rand(8192, K, generator=g, device="cuda") < 1e-3, blk * 100, blk)
        x[r0:r0 + 8192] = blk.to(torch.bfloat16)
    q, s = _quant(x, column_major_scales=True, scale_tma_aligned=True)
    q_rm, s_rm = _quant(x)
    assert same_bits(q, q_rm) and same_bits(s.contiguous(), s_rm)
    rows = torch.arange(0, M, 509)
    q_ref, s_ref = O.quant_group_fp8_cuda_semantics(x[rows.cuda()].cpu(), 128)
    assert same_bits(q[rows.cuda()].cpu(), q_ref) and same_bits(s[rows.cuda()].contiguous().cpu(), s_ref)
    for r0 in range(0, M, 8192):
        xf = x[r0:r0 + 8192].float().view(8192, K // 128, 128)
        amax_t = xf.abs().amax(-1).clamp(min=1e-10)
        s_t = amax_t / torch.full_like(amax_t, 448.0)   # tensor / tensor: an IEEE division (a Python-scalar divisor becomes a reciprocal multiply on CUDA)
        q_t = (xf / s_t.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(8192, K)
        assert same_bits(q_rm[r0:r0 + 8192], q_t) and same_bits(s_rm[r0:r0 + 8192], s_t), r0
        if r0 == 0:   # the restatement itself against the oracle
            idx = rows[rows < 8192].cuda()
            n = idx.numel()
            assert same_bits(q_t[idx].cpu(), q_ref[:n]) and same_bits(s_t[idx].cpu(), s_ref[:n])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,K", [(1, 128), (5, 512), (37, 1024), (130, 7168), (2048, 7168), (6, 640)])
def test_ue8m0_packed_scales_bit_exact(M, K, dtype):
    """scale_ue8m0=True: power-of-two scales as packed exponent bytes (int32, column-major, padded to 4 rows and
    4 groups), codes and words bit-exact against the oracle; padding rows / words stay zero."""
    x = O.gen_activation(M, K, seed=M + K, dtype=dtype, outlier_frac=1e-3)
    q, s = _quant(x, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
    q_ref, s_ref, packed_ref = O.quant_group_fp8_ue8m0_cuda_semantics(x, 128)
    words = (K // 128 + 3) // 4
    assert s.dtype == torch.int32 and tuple(s.shape) == (M, words) and s.stride(0) == 1
    assert s.stride(1) == (M + 3) // 4 * 4
    assert count_diff_bits(q.cpu(), q_ref) == 0
    assert torch.equal(s.cpu(), packed_ref)
    storage = torch.as_strided(s, (words, s.stride(1)), (s.stride(1), 1)).cpu()
    assert bool((storage[:, M:] == 0).all())


def test_ue8m0_golden_and_edge_cases():
    g = load_golden("quant_ue8m0.npz")
    x = as_bf16(g["x"])
    q, s = _quant(x, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
    assert same_bits(q.cpu(), as_fp8(g["xq"]))
    sf = t(g["xs"])
    by = torch.stack([(s.cpu() >> (8 * b)) & 0xFF for b in range(4)], dim=-1).reshape(x.shape[0], -1)
    assert torch.equal(torch.pow(2.0, (by[:, :sf.shape[1]] - 127).float()), sf)
    # an all-zero group: amax = eps -> scale 2**ceil(log2(1e-10)) = 2**-33 (byte 94), codes zero;
    # exact powers of two times 448 keep their exponent (ceil of an integer)
    z = torch.zeros(2, 256, dtype=torch.bfloat16)
    z[1, :128] = 448.0 * 2.0 ** -3
    z[1, 128:] = 448.0 * 2.0 ** 5
    qz, sz = _quant(z, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
    qr, sr, pr = O.quant_group_fp8_ue8m0_cuda_semantics(z, 128)
    assert torch.equal(sz.cpu(), pr) and count_diff_bits(qz.cpu(), qr) == 0
    assert int(sz[0, 0]) & 0xFF == 94 and int(sz[1, 0]) & 0xFF == 124 and (int(sz[1, 0]) >> 8) & 0xFF == 132


def test_ue8m0_argument_errors():
    from sglang_b200.sgl_kernel import sgl_per_token_group_quant_fp8
    x = torch.randn(8, 256, device="cuda").to(torch.bfloat16)
    q = torch.empty(8, 256, device="cuda", dtype=torch.float8_e4m3fn)
    with pytest.raises(RuntimeError):      # fp32 scale tensor with scale_ue8m0
        sgl_per_token_group_quant_fp8(x, q, torch.empty(8, 2, device="cuda"), 128, 1e-10, -448.0, 448.0, True)
    with pytest.raises(RuntimeError):      # row-major int32
        sgl_per_token_group_quant_fp8(x, q, torch.zeros(8, 2, device="cuda", dtype=torch.int32)[:, :1], 128, 1e-10,
                                      -448.0, 448.0, True)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("with_residual", [False, True])
@pytest.mark.parametrize("M,K", [(1, 128), (19, 1024), (64, 7168), (5, 16384), (300, 8192)])
def test_rmsnorm_alone_against_the_oracle(M, K, with_residual, dtype):
    """The norm kernel against RMSNorm.forward_native's arithmetic (the oracle, pinned to the reference's method by
    tests/golden/rmsnorm_native.npz).  The only freedom is the order of the fp32 sum of squares (and rsqrt's last
    bit): an element may differ by one unit in the last place of the 16-bit type; the residual sum must be exact."""
    from sglang_b200.layers.quantization.fp8_kernel import rmsnorm
    g = torch.Generator().manual_seed(M + K)
    x = (torch.randn(M, K, generator=g) * 2).to(dtype)
    w = (1.0 + 0.1 * torch.randn(K, generator=g)).to(dtype)
    r = torch.randn(M, K, generator=g).to(dtype) if with_residual else None
    if with_residual:
        y_ref, r_ref = O.rmsnorm_native(x, w, 1e-6, r)
        r_dev = r.cuda()
        y = rmsnorm(x.cuda(), w.cuda(), 1e-6, residual=r_dev).cpu()
        assert same_bits(r_dev.cpu(), r_ref)
    else:
        y_ref = O.rmsnorm_native(x, w, 1e-6)
        y = rmsnorm(x.cuda(), w.cuda(), 1e-6).cpu()
    ulp = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
    diff = (y.float() - y_ref.float()).abs()
    assert (diff <= ulp * y_ref.float().abs() + 1e-30).all()
    assert (diff == 0).float().mean() > 0.99


@pytest.mark.parametrize("layout", ["row", "col_tma", "ue8m0"])
@pytest.mark.parametrize("with_residual", [False, True])
@pytest.mark.parametrize("M,K", [(1, 128), (37, 1024), (64, 7168), (130, 2048)])
def test_rmsnorm_quant_fused_equals_the_two_kernel_sequence(M, K, with_residual, layout):
    """One pass == norm kernel, then the quant kernel: codes, scales, normalised rows and residual, bit for bit."""
    from sglang_b200.layers.quantization.fp8_kernel import (rmsnorm, rmsnorm_per_token_group_quant_fp8,
                                                            sglang_per_token_group_quant_fp8)
    g = torch.Generator().manual_seed(M * 3 + K)
    x = O.gen_activation(M, K, seed=M, outlier_frac=1e-3).cuda()
    w = (1.0 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16).cuda()
    r0 = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda() if with_residual else None
    kw = {"row": {}, "col_tma": dict(column_major_scales=True, scale_tma_aligned=True),
          "ue8m0": dict(column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)}[layout]
    r1 = r0.clone() if with_residual else None
    y = rmsnorm(x, w, 1e-6, residual=r1)
    q_ref, s_ref = sglang_per_token_group_quant_fp8(y, 128, **kw)
    r2 = r0.clone() if with_residual else None
    q, s, y2 = rmsnorm_per_token_group_quant_fp8(x, w, 1e-6, residual=r2, return_normed=True, **kw)
    assert same_bits(y2.cpu(), y.cpu())
    assert same_bits(q.cpu(), q_ref.cpu()) and torch.equal(s.cpu(), s_ref.cpu())
    assert s.stride() == s_ref.stride()
    if with_residual:
        assert same_bits(r2.cpu(), r1.cpu())
    q3, s3 = rmsnorm_per_token_group_quant_fp8(x, w, 1e-6, residual=r0.clone() if with_residual else None, **kw)
    assert same_bits(q3.cpu(), q_ref.cpu()) and torch.equal(s3.cpu(), s_ref.cpu())


# ------------------------------------------------------------------------------------------ int8 destination
def _check_int8(x, group=128, column_major=False):
    from sglang_b200.sgl_kernel import sgl_per_token_group_quant_int8
    xd = x.cuda()
    M, K = x.shape
    q = torch.empty(M, K, dtype=torch.int8, device="cuda")
    s = (torch.empty(K // group, M, device="cuda").t() if column_major else torch.empty(M, K // group, device="cuda"))
    sgl_per_token_group_quant_int8(xd, q, s, group, 1e-10, -128, 127)
    q_ref, s_ref = O.quant_group_int8_cuda_semantics(x, group)
    assert torch.equal(q.cpu(), q_ref), f"{(q.cpu() != q_ref).sum().item()} codes differ of {q_ref.numel()}"
    assert same_bits(s.cpu().contiguous(), s_ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("group", [64, 128, 256, 512])
@pytest.mark.parametrize("shape", [(1, 512), (7, 512), (83, 4096), (33, 5120), (2048, 7168)])
def test_int8_destination_bit_exact(shape, group, dtype):
    """The reference's own grid for the int8 form (sgl-kernel/tests/test_per_token_group_quant_8bit.py:268-276):
    codes (truncated toward zero) and scales against the oracle, both scale layouts."""
    g = torch.Generator().manual_seed(shape[0] * 31 + group)
    x = (torch.randn(shape, generator=g) * torch.where(torch.rand(shape, generator=g) < 1e-3, 100.0, 1.0)).to(dtype)
    _check_int8(x, group)
    _check_int8(x, group, column_major=True)


def test_int8_destination_golden_and_special_values():
    from sglang_b200.layers.quantization.int8_kernel import sglang_per_token_group_quant_int8
    g = load_golden("quant_int8_native.npz")
    x = as_bf16(g["bf16_x"])
    q, s = sglang_per_token_group_quant_int8(x.cuda(), 128)
    assert torch.equal(q.cpu(), torch.from_numpy(g["bf16_g128_q"]))
    assert same_bits(s.cpu(), t(g["bf16_g128_s"]).reshape(s.shape))
    x = torch.zeros(8, 256, dtype=torch.bfloat16)
    x[1, 5] = float("nan"); x[1, 7] = 3.0
    x[2, 0] = float("inf"); x[2, 1] = 1.0
    x[3, :128] = 1e-30
    x[4, 3] = -65280.0; x[4, 4] = 2.0 ** -120
    x[5, 130] = -0.0
    x[6, :] = torch.finfo(torch.bfloat16).max
    x[7, ::2] = 0.999; x[7, 1] = 127.0          # quotients just below an integer: truncation, not rounding
    _check_int8(x)
    # a scale whose significand is all ones takes the literal division
    xf = torch.randn(64, 256).clamp(-1.0, 1.0)
    xf[:, 0] = float(np.float32(127.0) * np.frombuffer(np.uint32(0x3fffffff).tobytes(), dtype=np.float32)[0])
    _check_int8(xf)
    empty_q, empty_s = sglang_per_token_group_quant_int8(torch.empty(0, 256, dtype=torch.bfloat16, device="cuda"), 128)
    assert empty_q.shape == (0, 256) and empty_s.shape == (0, 2)


def test_int8_destination_full_size_property():
    """The benchmark's quantisation size (16384 x 7168): dequantised codes lie within one step below the input in
    magnitude (truncation never rounds away from zero), and every group's largest code is 127 or -- where
    amax / (amax / 127) rounds just below 127 -- 126."""
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(16384, 7168, generator=g, device="cuda").to(torch.bfloat16)
    from sglang_b200.layers.quantization.int8_kernel import sglang_per_token_group_quant_int8
    q, s = sglang_per_token_group_quant_int8(x, 128)
    xf = x.float().view(16384, 56, 128)
    deq = q.float().view(16384, 56, 128) * s.unsqueeze(-1)
    assert bool((deq.abs() <= xf.abs() * (1 + 1e-6)).all())
    assert bool(((xf - deq).abs() <= s.unsqueeze(-1) * (1 + 1e-6)).all())
    assert bool((q.view(16384, 56, 128).to(torch.int16).abs().amax(dim=-1) >= 126).all())

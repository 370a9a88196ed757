"""GPU parity: dense block-scaled FP8 GEMM against the CPU oracle.

Acceptance (stated tolerance): rel-L2 <= 1e-3 of (i) the kernel's fp32 result vs the oracle's
fp32 result and (ii) the bf16 output vs the oracle result rounded to bf16; (iii) bf16 output vs
the unrounded fp32 oracle sits at the bf16 format floor (about 1.7e-3) for any implementation
and is not asserted.  Shapes follow sgl-kernel/tests/test_fp8_blockwise_gemm.py
:84-89, python/sglang/test/test_block_fp8.py:340-357 and the benchmark configurations.
"""
import pytest
import torch

from oracle import block_fp8_oracle as O
from helpers import as_bf16, as_fp8, load_golden, same_bits, t

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn
TOL = 1e-3


def _rand_problem(M, N, K, seed, scale_kind="quant"):
    g = torch.Generator().manual_seed(seed)
    if scale_kind == "quant":
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        a, sa = O.quant_group_fp8_cuda_semantics(x, 128)
        w = torch.randn(N, K, generator=g) * 0.02
        b, sb = O.per_block_cast_to_fp8(w)
    else:  # sgl-kernel test distribution: U(-448,448) codes, randn*1e-3 scales
        a = ((torch.rand(M, K, generator=g) - 0.5) * 2 * 448).to(FP8)
        b = ((torch.rand(N, K, generator=g) - 0.5) * 2 * 448).to(FP8)
        sa = torch.randn(M, K // 128, generator=g) * 1e-3
        sb = torch.randn((N + 127) // 128, K // 128, generator=g) * 1e-3
    return a, b, sa.contiguous(), sb.contiguous()


def _run_sgl(a, b, sa, sb, out_dtype=torch.bfloat16):
    from sglang_b200.sgl_kernel import fp8_blockwise_scaled_mm
    sa_d = sa.cuda().t().contiguous().t()          # M-major
    sb_d = sb.cuda().t()                           # [K/128, N/128], K-major (stride(0) == 1)
    return fp8_blockwise_scaled_mm(a.cuda(), b.cuda().t(), sa_d, sb_d, out_dtype)


def _run_w8a8(a, b, sa, sb, out_dtype):
    from sglang_b200.layers.quantization.fp8_kernel import w8a8_block_fp8_matmul
    return w8a8_block_fp8_matmul(a.cuda(), b.cuda(), sa.cuda(), sb.cuda(), [128, 128], out_dtype)


def _status_ok():
    import ctypes
    from sglang_b200 import _lib
    st = ctypes.c_int(0)
    _lib.check("status", _lib.lib().b200_gemm_device_status(ctypes.byref(st)))
    assert st.value == 0, f"device status word = {st.value}"
    # the host mirror (read without a synchronisation) agrees
    _lib.check("poll", _lib.lib().b200_gemm_poll_status(ctypes.byref(st)))
    assert st.value == 0, f"host mirror of the status word = {st.value}"


def _assert_parity(a, b, sa, sb, force_block_n=0):
    from sglang_b200 import _lib
    _lib.lib().b200_debug_force_block_n(force_block_n)
    try:
        ref32 = O.block_fp8_matmul_fp32(a, b, sa, sb)
        c32 = _run_w8a8(a, b, sa, sb, torch.float32).cpu()
        cbf = _run_w8a8(a, b, sa, sb, torch.bfloat16).cpu()
        _status_ok()
    finally:
        _lib.lib().b200_debug_force_block_n(0)
    e32 = O.rel_l2(c32, ref32)
    ebf = O.rel_l2(cbf.float(), ref32.to(torch.bfloat16).float())
    assert e32 <= TOL and ebf <= TOL, (e32, ebf)
    return c32, cbf


@pytest.fixture
def no_split_k():
    """Runs the unsplit kernel even for decode-size batches."""
    from sglang_b200.sgl_kernel import gemm
    gemm.SPLIT_K_MODE = "off"
    yield
    gemm.SPLIT_K_MODE = "auto"


@pytest.mark.parametrize("block_n", [128, 256, 3, 3032])   # 3xxx = weight-streaming kernel
@pytest.mark.parametrize("K", [128, 256, 512, 1024])
@pytest.mark.parametrize("N", [128, 256, 512, 1152])
@pytest.mark.parametrize("M", [1, 3, 5, 127, 128, 129, 512])
def test_small_grid(M, N, K, block_n, no_split_k):
    a, b, sa, sb = _rand_problem(M, N, K, seed=M * 7 + N * 3 + K, scale_kind="uniform")
    _assert_parity(a, b, sa, sb, block_n)


# ---------------------------------------------------------------------------- split-K (small M)
def _run_splitk(a, b, sa, sb, out_dtype, split_k, ws_floats=None):
    """Straight through the C ABI with a forced split count."""
    from sglang_b200 import _lib
    from sglang_b200.sgl_kernel.gemm import _DT
    M, K = a.shape
    N = b.shape[0]
    ad, bd = a.cuda(), b.cuda()
    sad, sbd = sa.cuda().contiguous(), sb.cuda().contiguous()
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device="cuda")
    n_ws = split_k * M * N if ws_floats is None else ws_floats
    ws = torch.full((max(n_ws, 4),), float("nan"), dtype=torch.float32, device="cuda")
    rc = _lib.lib().b200_fp8_blockwise_scaled_mm_splitk(
        ad.data_ptr(), K, bd.data_ptr(), K, sad.data_ptr(), sad.stride(0), sad.stride(1),
        sbd.data_ptr(), sbd.stride(0), sbd.stride(1), out.data_ptr(), N, _DT[out_dtype], M, N, K,
        split_k, ws.data_ptr(), n_ws * 4, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, out


@pytest.mark.parametrize("block_n", [0, 128, 3, 3064])
@pytest.mark.parametrize("split_k", [2, 3, 5, 8])
@pytest.mark.parametrize("M,N,K", [(1, 512, 1024), (16, 384, 1152), (128, 1152, 2048), (77, 256, 4096),
                                   (5, 128, 1024)])
def test_split_k_forced(M, N, K, split_k, block_n):
    from sglang_b200 import _lib
    a, b, sa, sb = _rand_problem(M, N, K, seed=M + N + K + split_k, scale_kind="uniform")
    ref32 = O.block_fp8_matmul_fp32(a, b, sa, sb)
    _lib.lib().b200_debug_force_block_n(block_n)
    try:
        rc32, c32 = _run_splitk(a, b, sa, sb, torch.float32, split_k)
        rcbf, cbf = _run_splitk(a, b, sa, sb, torch.bfloat16, split_k)
    finally:
        _lib.lib().b200_debug_force_block_n(0)
    assert rc32 == 0 and rcbf == 0
    _status_ok()
    assert O.rel_l2(c32.cpu(), ref32) <= TOL
    assert O.rel_l2(cbf.cpu().float(), ref32.to(torch.bfloat16).float()) <= TOL


def test_split_k_is_deterministic_and_matches_unsplit_to_rounding():
    a, b, sa, sb = _rand_problem(32, 1024, 4096, seed=5)
    _, c1 = _run_splitk(a, b, sa, sb, torch.float32, 1)
    _, c4a = _run_splitk(a, b, sa, sb, torch.float32, 4)
    _, c4b = _run_splitk(a, b, sa, sb, torch.float32, 4)
    assert same_bits(c4a, c4b)
    assert O.rel_l2(c4a.cpu(), c1.cpu()) <= 1e-6


@pytest.mark.parametrize("M", [1, 16, 64, 128, 256])
@pytest.mark.parametrize("N,K", [(7168, 18432), (36864, 7168), (1536, 7168)])
def test_split_k_auto_decode_shapes(M, N, K):
    """DeepSeek-V3 down / gate_up / q_a projections at decode-size batches through the
    reference-facing wrapper (which picks the split), against the oracle."""
    import ctypes
    from sglang_b200 import _lib
    a, b, sa, sb = _rand_problem(M, N, K, seed=M + N)
    ref32 = O.block_fp8_matmul_fp32(a, b, sa, sb)
    cbf = _run_sgl(a, b, sa, sb).cpu()
    _status_ok()
    assert O.rel_l2(cbf.float(), ref32.to(torch.bfloat16).float()) <= TOL
    s, nb = ctypes.c_int(0), ctypes.c_size_t(0)
    assert _lib.lib().b200_fp8_blockwise_scaled_mm_splitk_plan(M, N, K, 148, ctypes.byref(s), ctypes.byref(nb)) == 0
    assert nb.value == (s.value * M * N * 4 if s.value > 1 else 0)
    if M <= 64:          # one token tile: narrow projections leave SMs idle and are split
        assert (s.value > 1) == (N <= 148 * 128)


def test_split_k_argument_errors():
    from sglang_b200 import _lib
    a, b, sa, sb = _rand_problem(8, 256, 1024, seed=1)
    rc, _ = _run_splitk(a, b, sa, sb, torch.bfloat16, 4, ws_floats=4 * 8 * 256 - 1)   # workspace one float short
    assert rc < 0
    rc, _ = _run_splitk(a, b, sa, sb, torch.bfloat16, 9)                               # more splits than k-blocks
    assert rc < 0
    rc, _ = _run_splitk(a, b, sa, sb, torch.bfloat16, 65)
    assert rc < 0
    # automatic split with no room falls back to the unsplit kernel
    rc, out = _run_splitk(a, b, sa, sb, torch.bfloat16, 0, ws_floats=0)
    assert rc == 0 and bool(torch.isfinite(out.float()).all())


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(1, 128, 512), (127, 4096, 1024), (512, 1024, 4096), (1024, 14080, 512)])
def test_sgl_kernel_entry_reference_tolerance(M, N, K, out_dtype):
    """sgl-kernel/tests/test_fp8_blockwise_gemm.py:62-81: assert_close(rtol=0.02, atol=1)."""
    a, b, sa, sb = _rand_problem(M, N, K, seed=5, scale_kind="uniform")
    o1 = _run_sgl(a, b, sa, sb, out_dtype).cpu()
    o = O.baseline_scaled_mm(a, b.t(), sa, sb.t(), out_dtype)
    torch.testing.assert_close(o, o1, rtol=0.02, atol=1)
    _status_ok()


def test_golden_and_known_answer():
    g = load_golden("matmul_native.npz")
    a, b, As, Bs = as_fp8(g["a"]), as_fp8(g["b"]), t(g["As"]), t(g["Bs"])
    c32 = _run_w8a8(a, b, As, Bs, torch.float32).cpu()
    assert O.rel_l2(c32, t(g["c_f32"])) <= TOL
    cbf = _run_w8a8(a, b, As, Bs, torch.bfloat16).cpu()
    assert O.rel_l2(cbf.float(), as_bf16(g["c_bf16"]).float()) <= TOL
    k = load_golden("known_answer.npz")   # N = 320: not a multiple of 128 (test_fp8_kernel.py:15-17)
    A, A_q, A_s = t(k["A"]), as_fp8(k["A_q"]), t(k["A_s"])
    B, B_q, B_s = t(k["B"]), as_fp8(k["B_q"]), t(k["B_s"])
    C = _run_w8a8(A_q, B_q.T.contiguous(), A_s, B_s.T.contiguous(), torch.bfloat16).cpu()
    C_gt = A.to(torch.bfloat16) @ B.to(torch.bfloat16)
    torch.testing.assert_close(C, C_gt, atol=0.5, rtol=1e-4)
    _status_ok()


def test_config0_linear_end_to_end():
    """M=64, K=7168, N=4096: quant + GEMM through the linear glue vs the oracle linear."""
    from sglang_b200.layers.quantization.fp8_utils import w8a8_block_fp8_linear
    x = O.gen_activation(64, 7168, seed=0)
    wq, ws = O.gen_weight(4096, 7168, seed=1)
    out = w8a8_block_fp8_linear(x.cuda(), wq.cuda(), [128, 128], ws.cuda()).cpu()
    q, s = O.quant_group_fp8_cuda_semantics(x, 128)
    ref32 = O.block_fp8_matmul_fp32(q, wq, s, ws)
    assert out.dtype == torch.bfloat16 and out.shape == (64, 4096)
    assert O.rel_l2(out.float(), ref32.to(torch.bfloat16).float()) <= TOL
    assert O.mean_rel_err(out, ref32) < 3e-3       # bf16 floor; reference metric test_block_fp8.py:394-398
    bias = torch.randn(4096).to(torch.bfloat16)
    out_b = w8a8_block_fp8_linear(x.cuda().view(2, 32, 7168), wq.cuda(), [128, 128], ws.cuda(), bias=bias.cuda())
    assert out_b.shape == (2, 32, 4096)
    assert same_bits(out_b.view(64, 4096).cpu(), out + bias)
    _status_ok()


@pytest.mark.parametrize("N,K", [(36864, 7168), (7168, 18432)])
@pytest.mark.parametrize("M", [1, 16, 128])
def test_config1_small_m(M, N, K):
    a, b, sa, sb = _rand_problem(M, N, K, seed=1000 + M)
    _assert_parity(a, b, sa, sb)


def _gpu_ref_fp32(a, b, sa, sb):
    """Same formula as the oracle, evaluated with fp32 torch matmuls on the GPU (TF32 off);
    used only where the CPU oracle would take minutes, and itself spot-checked against it."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        M, K = a.shape
        N = b.shape[0]
        C = torch.zeros(M, N, device="cuda")
        sb_rows = sb.repeat_interleave(128, 0)[:N]
        for kb in range(K // 128):
            ak = a[:, kb * 128:(kb + 1) * 128].float()
            bk = b[:, kb * 128:(kb + 1) * 128].float()
            C += (ak @ bk.t()) * (sa[:, kb:kb + 1] * sb_rows[:, kb][None, :])
        return C
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


@pytest.mark.parametrize("M,N,K", [(4096, 7168, 18432), (4096, 36864, 7168), (1024, 36864, 7168),
                                   (16384, 7168, 18432), (16384, 36864, 7168), (8192, 8192, 8192)])
def test_config1_large_m(M, N, K):
    """The large-M benchmark shapes (up to M = 16384; 8192^3-ish = the Llama-3-70B o_proj at M = 8192): every
    output against an fp32 restatement on the GPU, every 257th row against the CPU oracle."""
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8, w8a8_block_fp8_matmul
    a, sa = sglang_per_token_group_quant_fp8(x, 128)
    wq, ws = O.gen_weight(N, K, seed=3)
    b, sb = wq.cuda(), ws.cuda()
    out = w8a8_block_fp8_matmul(a, b, sa, sb, [128, 128], torch.bfloat16)
    out2 = w8a8_block_fp8_matmul(a, b, sa, sb, [128, 128], torch.bfloat16)
    assert same_bits(out, out2), "not deterministic"
    ref = _gpu_ref_fp32(a, b, sa, sb)
    assert O.rel_l2(out.float().cpu(), ref.to(torch.bfloat16).float().cpu()) <= TOL
    rows = torch.arange(0, M, 257)
    ref_cpu = O.block_fp8_matmul_fp32(a[rows.cuda()].cpu(), wq, sa[rows.cuda()].cpu(), ws)
    assert O.rel_l2(out[rows.cuda()].float().cpu(), ref_cpu.to(torch.bfloat16).float()) <= TOL
    _status_ok()


def test_no_out_of_bounds_writes():
    """Guard rows/columns around the output keep their canary value."""
    from sglang_b200 import _lib
    M, N, K = 130, 384, 256
    a, b, sa, sb = _rand_problem(M, N, K, seed=9)
    ldo = N + 64
    buf = torch.full((M + 8, ldo), -7.0, dtype=torch.bfloat16, device="cuda")
    a_d, b_d, sa_d, sb_d = a.cuda(), b.cuda(), sa.cuda(), sb.cuda()
    rc = _lib.lib().b200_fp8_blockwise_scaled_mm(a_d.data_ptr(), K, b_d.data_ptr(), K, sa_d.data_ptr(), K // 128, 1,
                                                 sb_d.data_ptr(), K // 128, 1, buf.data_ptr(), ldo, 2, M, N, K,
                                                 torch.cuda.current_stream().cuda_stream)
    _lib.check("mm", rc)
    torch.cuda.synchronize()
    assert torch.all(buf[M:] == -7.0) and torch.all(buf[:, N:] == -7.0)
    ref = O.block_fp8_matmul_fp32(a, b, sa, sb).to(torch.bfloat16)
    assert O.rel_l2(buf[:M, :N].float().cpu(), ref.float()) <= TOL
    _status_ok()


def test_argument_errors_raise_before_launch():
    from sglang_b200.sgl_kernel import fp8_blockwise_scaled_mm
    a = torch.zeros(4, 256, dtype=FP8, device="cuda")
    b = torch.zeros(128, 256, dtype=FP8, device="cuda")
    sa = torch.ones(2, 4, device="cuda").t()
    sb = torch.ones(1, 2, device="cuda").t()
    fp8_blockwise_scaled_mm(a, b.t(), sa, sb, torch.bfloat16)
    with pytest.raises(RuntimeError, match="row major"):
        fp8_blockwise_scaled_mm(a.t().contiguous().t(), b.t(), sa, sb, torch.bfloat16)
    with pytest.raises(RuntimeError, match="column major"):
        fp8_blockwise_scaled_mm(a, b.t().contiguous(), sa, sb, torch.bfloat16)
    with pytest.raises(RuntimeError, match="Float8_e4m3fn"):
        fp8_blockwise_scaled_mm(a.view(torch.uint8), b.t(), sa, sb, torch.bfloat16)
    with pytest.raises(RuntimeError, match="out_dtype"):
        fp8_blockwise_scaled_mm(a, b.t(), sa, sb, torch.float32)
    with pytest.raises(RuntimeError, match="M major"):
        fp8_blockwise_scaled_mm(a, b.t(), torch.ones(4, 2, device="cuda"), sb, torch.bfloat16)
    with pytest.raises(RuntimeError, match="scales_b"):
        fp8_blockwise_scaled_mm(a, b.t(), sa, torch.ones(3, 1, device="cuda"), torch.bfloat16)
    assert fp8_blockwise_scaled_mm(a[:0], b.t(), sa[:0], sb, torch.bfloat16).shape == (0, 128)


@pytest.mark.parametrize("N,K", [(1280, 8192), (7168, 8192), (8192, 1024), (8192, 3584), (10240, 8192)])
def test_llama70b_tp_shard_shapes(N, K):
    """Per-rank shapes of the Llama-3-70B layers at tp=8 (and qkv at tp=1): column-parallel shards
    split N, row-parallel shards split K; M = 128."""
    a, b, sa, sb = _rand_problem(128, N, K, seed=N + K)
    _assert_parity(a, b, sa, sb)


def test_fp8_linear_method_apply():
    """Fp8LinearMethod owning a merged column-parallel shard: create -> load -> apply vs the oracle linear."""
    from sglang_b200.layers.quantization.fp8 import Fp8Config, Fp8LinearMethod
    cfg = Fp8Config.from_config({"quant_method": "fp8", "activation_scheme": "dynamic", "weight_block_size": [128, 128]})
    method = Fp8LinearMethod(cfg)
    layer = torch.nn.Module()
    method.create_weights(layer, 1024, [256, 256], 1024, 4096, torch.bfloat16, tp_size=8, device="cuda")
    wq, ws = O.gen_weight(512, 1024, seed=3)
    layer.weight.data.copy_(wq.cuda())
    layer.weight_scale_inv.data.copy_(ws.cuda())
    method.process_weights_after_loading(layer)
    x = O.gen_activation(48, 1024, seed=4)
    bias = torch.randn(512).to(torch.bfloat16)
    out = method.apply(layer, x.cuda().view(3, 16, 1024), bias.cuda()).cpu()
    ref = O.block_fp8_linear(x, wq, ws, bias=bias)
    assert out.shape == (3, 16, 512) and out.dtype == torch.bfloat16
    assert O.rel_l2(out.view(48, 512).float(), ref.float()) <= TOL
    _status_ok()


@pytest.mark.parametrize("with_bias", [False, True])
def test_fp8_linear_method_apply_ragged_n(with_bias):
    """DeepSeek-V3's kv_a_proj_with_mqa: N = 576 is not a multiple of 128, its scales are ceil-sized [5, 56].
    The reference sends such layers to its Triton linear (fp8_utils.py:190-197); here the same CUDA kernel
    masks the ragged last block."""
    from sglang_b200.layers.quantization.fp8 import Fp8Config, Fp8LinearMethod
    cfg = Fp8Config.from_config({"quant_method": "fp8", "activation_scheme": "dynamic", "weight_block_size": [128, 128]})
    method = Fp8LinearMethod(cfg)
    layer = torch.nn.Module()
    N, K = 576, 7168
    method.create_weights(layer, K, [N], K, N, torch.bfloat16, tp_size=1, device="cuda")
    wq, ws = O.gen_weight(N, K, seed=31)
    assert tuple(layer.weight_scale_inv.shape) == tuple(ws.shape) == (5, 56)
    layer.weight.data.copy_(wq.cuda())
    layer.weight_scale_inv.data.copy_(ws.cuda())
    method.process_weights_after_loading(layer)
    for M in (1, 48, 200):
        x = O.gen_activation(M, K, seed=32 + M)
        bias = torch.randn(N, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16) if with_bias else None
        out = method.apply(layer, x.cuda(), bias.cuda() if with_bias else None).cpu()
        ref = O.block_fp8_linear(x, wq, ws, bias=bias)
        assert out.shape == (M, N) and out.dtype == torch.bfloat16
        assert O.rel_l2(out.float(), ref.float()) <= TOL
    _status_ok()


def test_out_argument_writes_a_row_slice_only():
    """`out=` (an extension of fp8_blockwise_scaled_mm and w8a8_block_fp8_linear): the result lands in a
    row slice of a larger buffer, bit-identical to the allocating call; neighbouring rows keep their value."""
    from sglang_b200.layers.quantization.fp8_utils import w8a8_block_fp8_linear
    M, N, K = 640, 1024, 2048
    x = O.gen_activation(M, K, seed=41).cuda()
    wq, ws = O.gen_weight(N, K, seed=42)
    wq, ws = wq.cuda(), ws.cuda()
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    want = w8a8_block_fp8_linear(x, wq, [128, 128], ws, bias=bias)
    buf = torch.full((3 * M, N), -7.0, dtype=torch.bfloat16, device="cuda")
    got = w8a8_block_fp8_linear(x, wq, [128, 128], ws, bias=bias, out=buf[M:2 * M])
    torch.cuda.synchronize()
    assert got.data_ptr() == buf[M:2 * M].data_ptr()
    assert same_bits(buf[M:2 * M], want)
    assert torch.all(buf[:M] == -7.0) and torch.all(buf[2 * M:] == -7.0)
    _status_ok()


# ---------------------------------------------------------------------------- packed UE8M0 activation scales
@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (16, 512, 1024), (64, 1152, 640), (130, 256, 7168), (512, 384, 1024)])
def test_ue8m0_scaled_matmul(M, N, K, no_split_k):
    """Activation scales as packed exponent bytes (what the quant op writes with scale_ue8m0=True), weights
    with power-of-two block scales: equal to the (unsplit) fp32-scale kernel given the decoded scales, bit for
    bit, and within tolerance of the oracle."""
    from sglang_b200.layers.quantization.fp8_kernel import (sglang_per_token_group_quant_fp8,
                                                            w8a8_block_fp8_matmul_deepgemm)
    x = O.gen_activation(M, K, seed=M + K, outlier_frac=1e-3)
    w = torch.randn(N, K, generator=torch.Generator().manual_seed(N)) * 0.02
    wq, ws = O.per_block_quant_mxfp8(w)
    q_ref, s_ref, packed_ref = O.quant_group_fp8_ue8m0_cuda_semantics(x, 128)
    q, s_packed = sglang_per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True, scale_tma_aligned=True,
                                                   scale_ue8m0=True)
    assert torch.equal(s_packed.cpu(), packed_ref)
    out = w8a8_block_fp8_matmul_deepgemm(q, wq.cuda(), s_packed, ws.cuda(), [128, 128], torch.bfloat16).cpu()
    _status_ok()
    ref32 = O.block_fp8_matmul_fp32(q_ref, wq, s_ref, ws)
    assert O.rel_l2(out.float(), ref32.to(torch.bfloat16).float()) <= TOL
    same = _run_w8a8(q_ref, wq, s_ref, ws, torch.bfloat16).cpu()
    assert same_bits(out, same)


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (128, 256, 512), (130, 512, 1024), (300, 1152, 640),
                                   (1024, 7168, 2048), (4096, 4096, 7168)])
def test_power_of_two_scales_on_the_block_scaling_mma(M, N, K):
    """Both scale sets powers of two (activations: packed UE8M0 from the quantiser; weights: per_block_quant_mxfp8):
    the hardware block-scaled product against the oracle's fp32 result and against the fp32-promotion kernel fed
    the same codes and scales.  Rows and weight blocks carry very different exponents (an activation row scaled by
    2^(row % 13), weight blocks by 2^(block index % 7)), so a scale applied to the wrong row, column block or
    k-block cannot pass."""
    from sglang_b200.layers.quantization.fp8_kernel import (sglang_per_token_group_quant_fp8,
                                                            w8a8_block_fp8_matmul_deepgemm)
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g)
    x = (x * torch.pow(2.0, (torch.arange(M) % 13).float()).unsqueeze(1)).to(torch.bfloat16)
    x[:, : K // 2] *= 4.0      # k-blocks of one row differ as well
    w = torch.randn(N, K, generator=g) * 0.02
    blk = (torch.arange((N + 127) // 128).unsqueeze(1) * (K // 128) + torch.arange(K // 128).unsqueeze(0)) % 7
    w = w * torch.pow(2.0, blk.float()).repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)
    wq, ws = O.per_block_quant_mxfp8(w)
    q_ref, s_ref, packed_ref = O.quant_group_fp8_ue8m0_cuda_semantics(x, 128)
    q, s_packed = sglang_per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True, scale_tma_aligned=True,
                                                   scale_ue8m0=True)
    from sglang_b200 import _lib
    ref32 = O.block_fp8_matmul_fp32(q_ref, wq, s_ref, ws)
    soft = w8a8_block_fp8_matmul_deepgemm(q, wq.cuda(), s_packed, ws.cuda(), [128, 128], torch.bfloat16).cpu()
    # 128 x 256 (one accumulator), 128 x 240 (two), 256 x 240 (two row halves), 256 x 256 on a CTA pair
    for tile_width in (0, 240, 2240, 2256):
        _lib.lib().b200_debug_force_block_n(tile_width)
        try:
            out = w8a8_block_fp8_matmul_deepgemm(q, wq.cuda(), s_packed, ws.cuda(), [128, 128], torch.bfloat16,
                                                 weight_scale_ue8m0=True).cpu()
            _status_ok()
        finally:
            _lib.lib().b200_debug_force_block_n(0)
        assert O.rel_l2(out.float(), ref32.to(torch.bfloat16).float()) <= TOL, tile_width
        assert O.rel_l2(out.float(), soft.float()) <= TOL, tile_width


def test_fp8_linear_method_ue8m0_mode():
    """Fp8LinearMethod(scale_ue8m0=True): the weights are re-quantised to power-of-two block scales after loading
    (the arithmetic of the reference's requant_weight_ue8m0, pinned here by the oracle's per_block_quant_mxfp8 on
    the dequantised weight) and apply() runs the block-scaling MMA; against the oracle on the re-quantised weight."""
    from sglang_b200.layers.quantization.fp8 import Fp8Config, Fp8LinearMethod
    cfg = Fp8Config.from_config({"quant_method": "fp8", "activation_scheme": "dynamic", "weight_block_size": [128, 128]})
    method = Fp8LinearMethod(cfg, scale_ue8m0=True)
    layer = torch.nn.Module()
    N, K, M = 512, 1024, 96
    method.create_weights(layer, K, [N], K, N, torch.bfloat16, tp_size=1, device="cuda")
    wq, ws = O.gen_weight(N, K, seed=51)
    layer.weight.data.copy_(wq.cuda())
    layer.weight_scale_inv.data.copy_(ws.cuda())
    method.process_weights_after_loading(layer)
    w_deq = (wq.float() * ws.repeat_interleave(128, 0).repeat_interleave(128, 1)).to(torch.bfloat16)
    wq2, ws2 = O.per_block_quant_mxfp8(w_deq)
    assert same_bits(layer.weight.data.cpu(), wq2) and torch.equal(layer.weight_scale_inv.data.cpu(), ws2)
    assert bool((torch.log2(ws2) == torch.log2(ws2).round()).all())
    x = O.gen_activation(M, K, seed=52)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(53)).to(torch.bfloat16)
    out = method.apply(layer, x.cuda(), bias.cuda()).cpu()
    q_ref, s_ref, _ = O.quant_group_fp8_ue8m0_cuda_semantics(x, 128)
    ref = O.block_fp8_matmul_fp32(q_ref, wq2, s_ref, ws2).to(torch.bfloat16) + bias
    assert O.rel_l2(out.float(), ref.float()) <= TOL
    _status_ok()


def test_deepgemm_shaped_linear():
    """deepgemm_w8a8_block_fp8_linear_with_fallback: quantise with packed power-of-two scales, multiply, add
    bias, view back; the fp32-scale fallback for shapes the DeepGEMM path does not take."""
    from sglang_b200.layers.quantization.fp8_utils import deepgemm_w8a8_block_fp8_linear_with_fallback as lin
    x = O.gen_activation(48, 1024, seed=11)
    w = torch.randn(512, 1024, generator=torch.Generator().manual_seed(12)) * 0.02
    wq, ws = O.per_block_quant_mxfp8(w)
    bias = torch.randn(512).to(torch.bfloat16)
    out = lin(x.cuda().view(3, 16, 1024), wq.cuda(), [128, 128], ws.cuda(), bias=bias.cuda()).cpu()
    q_ref, s_ref, _ = O.quant_group_fp8_ue8m0_cuda_semantics(x, 128)
    ref = O.block_fp8_matmul_fp32(q_ref, wq, s_ref, ws).to(torch.bfloat16) + bias
    assert out.shape == (3, 16, 512)
    assert O.rel_l2(out.view(48, 512).float(), ref.float()) <= TOL
    # fp16 activations are not a DeepGEMM case: falls back to the fp32-scale linear
    out16 = lin(x.to(torch.float16).cuda(), wq.cuda(), [128, 128], ws.cuda()).cpu()
    ref16 = O.block_fp8_linear(x.to(torch.float16), wq, ws, out_dtype=torch.float16)
    assert out16.dtype == torch.float16 and O.rel_l2(out16.float(), ref16.float()) <= TOL
    _status_ok()


# ---------------------------------------------------------------------------- tail split (large M)
@pytest.mark.parametrize("M,N,K", [(4096, 7168, 2048), (4100, 7168, 2048), (8192, 1280, 4096), (4096, 7040, 2176)])
def test_tail_split_large_m(M, N, K):
    """Shapes whose last wave of tiles is mostly empty: the wrapper asks the plan, the library splits only
    those tiles' k-blocks.  Equal to the unsplit kernel to fp32 rounding (bit-identical outside the tail
    tiles), deterministic, within tolerance of the fp32 reference; M and N need not be tile multiples."""
    import ctypes
    from sglang_b200 import _lib
    from sglang_b200.sgl_kernel import gemm as G
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8, w8a8_block_fp8_matmul
    s, nb = ctypes.c_int(0), ctypes.c_size_t(0)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert _lib.lib().b200_fp8_blockwise_scaled_mm_splitk_plan(M, N, K, sms, ctypes.byref(s), ctypes.byref(nb)) == 0
    if sms == 148:
        assert s.value > 1 and nb.value > 0, "the case is meant to have a mostly empty last wave"
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    a, sa = sglang_per_token_group_quant_fp8(x, 128)
    wq, ws = O.gen_weight((N + 127) // 128 * 128, K, seed=5)
    b, sb = wq[:N].contiguous().cuda(), ws.cuda()
    out = w8a8_block_fp8_matmul(a, b, sa, sb, [128, 128], torch.bfloat16)
    out2 = w8a8_block_fp8_matmul(a, b, sa, sb, [128, 128], torch.bfloat16)
    assert same_bits(out, out2), "not deterministic"
    G.SPLIT_K_MODE = "off"
    try:
        plain = w8a8_block_fp8_matmul(a, b, sa, sb, [128, 128], torch.bfloat16)
    finally:
        G.SPLIT_K_MODE = "auto"
    _status_ok()
    ref = _gpu_ref_fp32(a, b, sa, sb)
    assert O.rel_l2(out.float().cpu(), ref.to(torch.bfloat16).float().cpu()) <= TOL
    assert O.rel_l2(out.float().cpu(), plain.float().cpu()) <= 2e-4      # a bf16 ulp here and there in the tail tiles
    if s.value > 1:
        differing_rows = int((out != plain).any(dim=1).sum())
        assert differing_rows <= 128 * 74, differing_rows   # only tail tiles (at most half a wave) may differ at all


def test_sm_limit_changes_the_grid_not_the_result():
    """b200_set_sm_limit: the persistent kernels run on fewer SMs (what a row-parallel linear does to leave SMs to
    its all-reduce); same bits, and the previous limit comes back from the call."""
    from sglang_b200.sgl_kernel.gemm import set_sm_limit
    a, b, sa, sb = _rand_problem(700, 1280, 2048, seed=5)
    full = _run_sgl(a, b, sa, sb).cpu()
    assert set_sm_limit(100) == 0
    try:
        limited = _run_sgl(a, b, sa, sb).cpu()
        _status_ok()
    finally:
        assert set_sm_limit(0) == 100
    assert same_bits(limited, full)

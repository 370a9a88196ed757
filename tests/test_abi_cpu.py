"""CPU: the C-ABI library loads, exports every symbol the header declares, and rejects bad
arguments with the documented codes before touching a device (no compute calls here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200_block_fp8.h")


def _declared():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", src)))


@pytest.fixture(scope="module")
def lib():
    from sglang_b200 import _lib
    if not os.path.isfile(_lib.LIB_PATH):
        from sglang_b200 import build
        build.build()
    return _lib.lib()


def test_every_declared_symbol_is_exported(lib):
    names = _declared()
    assert len(names) >= 14, names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_python_binding_lists_the_header(lib):
    from sglang_b200 import _lib
    bound = set(_lib.exported_symbols())
    assert set(_declared()) <= bound, sorted(set(_declared()) - bound)


def test_error_strings(lib):
    assert lib.b200_strerror(0) == b"ok"
    for code in range(-10, 0):
        assert lib.b200_strerror(code) not in (b"", b"unknown error code")
    assert lib.b200_strerror(-99) == b"unknown error code"
    assert lib.b200_abi_version() >= 1


def test_argument_checks_return_before_any_device_work(lib):
    P = ctypes.c_void_p
    one = P(16)     # an aligned, never dereferenced pointer value
    # quant: K not a multiple of the group, unsupported group, bad dtype, null pointers, misaligned
    q = lib.b200_per_token_group_quant_fp8
    assert q(one, 2, one, one, 4, 100, 128, 1, 1, 1e-10, -448.0, 448.0, None) == -3
    assert q(one, 2, one, one, 4, 192, 96, 2, 1, 1e-10, -448.0, 448.0, None) == -6
    assert q(one, 7, one, one, 4, 256, 128, 2, 1, 1e-10, -448.0, 448.0, None) == -2
    assert q(None, 2, one, one, 4, 256, 128, 2, 1, 1e-10, -448.0, 448.0, None) == -1
    assert q(P(8), 2, one, one, 4, 256, 128, 2, 1, 1e-10, -448.0, 448.0, None) == -5
    assert q(one, 2, one, one, 0, 256, 128, 2, 1, 1e-10, -448.0, 448.0, None) == 0       # M == 0: no-op
    q8 = lib.b200_per_token_group_quant_int8
    assert q8(one, 2, one, one, 4, 100, 128, 1, 1, 1e-10, -128.0, 127.0, None) == -3
    assert q8(one, 2, one, one, 4, 192, 96, 2, 1, 1e-10, -128.0, 127.0, None) == -6
    assert q8(None, 2, one, one, 4, 256, 128, 2, 1, 1e-10, -128.0, 127.0, None) == -1
    # GEMM: shapes, strides, alignment, dtype
    mm = lib.b200_fp8_blockwise_scaled_mm
    assert mm(one, 256, one, 256, one, 1, 4, one, 2, 1, one, 128, 2, -1, 128, 256, None) == -3
    assert mm(one, 256, one, 256, one, 1, 4, one, 2, 1, one, 128, 2, 0, 128, 256, None) == 0        # M == 0
    assert mm(None, 256, one, 256, one, 1, 4, one, 2, 1, one, 128, 2, 4, 128, 256, None) == -1
    assert mm(one, 256, one, 256, one, 1, 4, one, 2, 1, one, 128, 9, 4, 128, 256, None) == -2
    assert mm(one, 200, one, 256, one, 1, 4, one, 2, 1, one, 128, 2, 4, 128, 256, None) == -4      # lda < K
    assert mm(one, 264, one, 256, one, 1, 4, one, 2, 1, one, 128, 2, 4, 128, 256, None) == -5      # lda % 16
    # MoE glue
    assert lib.b200_shuffle_rows(None, one, one, 4, 64, None) == -1
    assert lib.b200_shuffle_rows(one, one, one, 0, 64, None) == 0
    assert lib.b200_silu_and_mul(one, one, 4, 12, 2, None) == -5                                   # d % 8
    assert lib.b200_apply_shuffle_mul_sum(one, one, one, None, 4, 0, 64, 2, None) == -3            # topk <= 0
    assert lib.b200_moe_prepare(one, 4, 2, 0, 8, 8, one, None, one, one, one, one, one, 64, None) == -3
    assert lib.b200_moe_prepare_scratch_bytes(32768, 256) == 16 * 256 * 4
    assert lib.b200_moe_prepare_noalloc(one, 2048 * 2048, 1, 64, 8, 8, one, None, one, one, one, one, None) == -9


def test_split_k_plan_needs_no_device(lib):
    """Decode-size batches on narrow, deep projections split; wide or shallow ones do not."""
    def plan(M, N, K, sms=148):
        s, b = ctypes.c_int(-1), ctypes.c_size_t(1)
        assert lib.b200_fp8_blockwise_scaled_mm_splitk_plan(M, N, K, sms, ctypes.byref(s), ctypes.byref(b)) == 0
        if M <= 512:
            assert b.value == (s.value * M * N * 4 if s.value > 1 else 0)
        return s.value
    assert plan(16, 7168, 18432) == 2          # <= 64 tokens: 56 tiles of 128 weight rows on 148 SMs
    assert plan(128, 7168, 18432) == 1         # 65..128 tokens: two token tiles x 56 weight tiles, 76 % of one wave
    assert plan(1, 1536, 7168) == 7            # capped at eight k-blocks per CTA
    assert plan(16, 36864, 7168) == 1          # already more tiles than SMs
    assert plan(16, 7168, 2048) == 1           # too few k-blocks to pay for the reduce kernel
    assert plan(129, 7168, 18432) == 2         # three token tiles x 56: 168 tiles, a nearly empty second wave
    assert plan(192, 10240, 8192) == 1         # 240 tiles: 81 % of two waves
    assert plan(256, 7168, 18432) == 2         # beyond 192 tokens 128 x 256 tiles: 56 of them
    assert plan(512, 7168, 18432) == 1         # 112 tiles: most SMs busy already
    assert plan(0, 7168, 18432) == 1
    assert plan(16, 7168, 18432, sms=0) == 2   # <= 0 means a 148-SM part
    # large M: only the last, mostly empty wave of tiles is split
    assert plan(4096, 7168, 18432) == 18       # 896 tiles of 128 x 256: six waves + 8 tiles -> 8 x 18 work units
    s, b = ctypes.c_int(0), ctypes.c_size_t(0)
    assert lib.b200_fp8_blockwise_scaled_mm_splitk_plan(4096, 7168, 18432, 148, ctypes.byref(s), ctypes.byref(b)) == 0
    assert b.value == 8 * 18 * 128 * 256 * 4
    assert plan(4096, 36864, 7168) == 7        # 4608 tiles: 31 waves + 20 tiles
    assert plan(16384, 36864, 7168) == 1       # 18432 tiles: the last wave is 80 tiles, more than half of the SMs
    assert plan(8192, 2560, 8192) == 3         # 640 tiles: four waves + 48 tiles -> 48 x 3 work units
    assert plan(8192, 1280, 8192) == 6         # 320 tiles: two waves + 24 tiles
    assert plan(4096, 7168, 1024) == 1         # too few k-blocks to divide
    s, b = ctypes.c_int(0), ctypes.c_size_t(0)
    assert lib.b200_fp8_blockwise_scaled_mm_splitk_plan(-1, 128, 128, 148, ctypes.byref(s), ctypes.byref(b)) < 0
    assert lib.b200_fp8_blockwise_scaled_mm_splitk_plan(1, 128, 128, 148, None, None) < 0


def test_missing_library_fails_loudly(monkeypatch):
    from sglang_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libb200_block_fp8.so")
    with pytest.raises(ImportError, match="no fallback"):
        _lib.lib()


def test_operator_schemas_and_shape_functions():
    """torch.ops.sgl_kernel.* carry the reference's schemas (sgl-kernel/csrc/common_extension.cc:111-119,
    192-207) and trace on meta tensors without a device."""
    import torch
    import sglang_b200.sgl_kernel  # noqa: F401  (registers the operators)
    ops = torch.ops.sgl_kernel
    schema = str(ops.fp8_blockwise_scaled_mm.default._schema)
    assert "Tensor mat_a, Tensor mat_b, Tensor scales_a, Tensor scales_b, ScalarType out_dtype" in schema
    assert "bool scale_ue8m0" in str(ops.sgl_per_token_group_quant_fp8.default._schema)
    assert "float int8_min, float int8_max" in str(ops.sgl_per_token_group_quant_int8.default._schema)
    assert "Tensor? blockscale_offsets" in str(ops.prepare_moe_input.default._schema)
    assert "Tensor gating_output, bool renormalize" in str(ops.topk_softmax.default._schema)
    fp8 = torch.float8_e4m3fn
    a = torch.empty(64, 7168, dtype=fp8, device="meta")
    b = torch.empty(4096, 7168, dtype=fp8, device="meta").t()
    sa = torch.empty(56, 64, device="meta").t()
    sb = torch.empty(32, 56, device="meta").t()
    out = ops.fp8_blockwise_scaled_mm(a, b, sa, sb, torch.bfloat16)
    assert out.device.type == "meta" and out.shape == (64, 4096) and out.dtype == torch.bfloat16
    x = torch.empty(64, 7168, dtype=torch.bfloat16, device="meta")
    q = torch.empty(64, 7168, dtype=fp8, device="meta")
    s = torch.empty(64, 56, device="meta")
    assert ops.sgl_per_token_group_quant_fp8(x, q, s, 128, 1e-10, -448.0, 448.0, False) is None

"""Generate tests/golden/*.npz by RUNNING the reference's own pure-torch functions.

The reference package cannot be imported as a whole in this environment
(`import sglang` needs IPython, `sgl_kernel` is not installed), but the oracle
functions its tests define are plain torch.  This script parses the reference
test files, extracts exactly those function definitions with `ast`, executes
them unmodified in a namespace that only provides torch, and stores their
inputs and outputs.  Nothing from the reference is copied into the repository;
only the numeric vectors are committed.

Sources executed (paths inside the reference checkout):
  python/sglang/test/test_block_fp8.py      native_per_token_group_quant_fp8,
                                            native_w8a8_block_fp8_matmul,
                                            torch_w8a8_block_fp8_moe
  sgl-kernel/tests/test_fp8_blockwise_gemm.py   baseline_scaled_mm
  sgl-kernel/tests/test_fp8_blockwise_moe.py    calc_diff, per_token_cast_to_fp8,
                                                per_block_cast_to_fp8
  test/srt/quant/test_fp8_kernel.py         TestFP8Base._make_A / _make_B (known-answer generators)
  python/sglang/test/test_block_fp8_deep_gemm_blackwell.py   ceil_to_ue8m0, per_token_group_quant_mxfp8,
                                            per_block_quant_mxfp8 (power-of-two scales)
  python/sglang/srt/layers/layernorm.py     RMSNorm.forward_native (producer of the linear's input)
  test/srt/quant/test_block_int8.py         native_per_token_group_quant_int8 (int8 destination of the quantiser)

Usage:  python tests/golden/make_golden.py --reference <reference checkout> [--only ue8m0|rmsnorm|int8]
"""
from __future__ import annotations

import argparse
import ast
import os
from typing import Optional, Tuple, Type

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
FP8 = torch.float8_e4m3fn


def _extract(path: str, names, ns: dict, inside_class: str | None = None):
    with open(path) as f:
        src = f.read()
    tree = ast.parse(src)
    body = tree.body
    if inside_class is not None:
        body = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == inside_class).body
    for node in body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            node.decorator_list = []  # drop @staticmethod
            mod = ast.Module(body=[node], type_ignores=[])
            exec(compile(mod, path, "exec"), ns)
    missing = [n for n in names if n not in ns]
    assert not missing, f"{path}: not found: {missing}"


def _np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == FP8:
        return t.view(torch.uint8).numpy()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy()
    return t.numpy()


class _SiluAndMul:
    """Stand-in with the arithmetic of SiluAndMul.forward_native (activation.py:60-62)."""
    def forward_native(self, x):
        d = x.shape[-1] // 2
        return F.silu(x[..., :d]) * x[..., d:]


def make_ue8m0(reference: str):
    """Power-of-two (UE8M0) scales: the reference's torch functions on seeded inputs."""
    ns = {"torch": torch, "Tuple": Tuple}
    _extract(os.path.join(reference, "python/sglang/test/test_block_fp8_deep_gemm_blackwell.py"),
             ["ceil_div", "align", "ceil_to_ue8m0", "per_token_group_quant_mxfp8", "per_block_quant_mxfp8"], ns)
    torch.manual_seed(7)
    x = (torch.randn(37, 1024) * torch.where(torch.rand(37, 1024) < 1e-2, 100.0, 1.0)).to(torch.bfloat16)
    xq, xs = ns["per_token_group_quant_mxfp8"](x)
    x32 = torch.randn(9, 384) * 3.0
    x32q, x32s = ns["per_token_group_quant_mxfp8"](x32)
    w = torch.randn(200, 384) * 0.02
    wq, ws = ns["per_block_quant_mxfp8"](w)
    np.savez_compressed(os.path.join(HERE, "quant_ue8m0.npz"), x=_np(x), xq=_np(xq), xs=_np(xs),
                        x32=_np(x32), x32q=_np(x32q), x32s=_np(x32s), w=_np(w), wq=_np(wq), ws=_np(ws))


def make_rmsnorm(reference: str):
    """RMSNorm.forward_native (python/sglang/srt/layers/layernorm.py:135-171), executed as written with a stand-in
    `self` that carries the four attributes the method reads."""
    from types import SimpleNamespace
    from typing import Union
    ns = {"torch": torch, "Optional": Optional, "Tuple": Tuple, "Union": Union}
    _extract(os.path.join(reference, "python/sglang/srt/layers/layernorm.py"), ["forward_native"], ns,
             inside_class="RMSNorm")
    out = {}
    for name, dtype in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        torch.manual_seed(11)
        x = (torch.randn(7, 512) * 2.0).to(dtype)
        r = torch.randn(7, 512).to(dtype)
        w = (1.0 + 0.1 * torch.randn(512)).to(dtype)
        me = SimpleNamespace(hidden_size=512, variance_size_override=None, variance_epsilon=1e-6, weight=w)
        y = ns["forward_native"](me, x.clone())
        y2, r2 = ns["forward_native"](me, x.clone(), r.clone())
        out.update({f"{name}_x": _np(x), f"{name}_r": _np(r), f"{name}_w": _np(w), f"{name}_y": _np(y),
                    f"{name}_y_res": _np(y2), f"{name}_r_out": _np(r2)})
    np.savez_compressed(os.path.join(HERE, "rmsnorm_native.npz"), **out)


def make_int8(reference: str):
    """native_per_token_group_quant_int8 (test/srt/quant/test_block_int8.py:13-35), executed as written."""
    ns = {"torch": torch}
    _extract(os.path.join(reference, "test/srt/quant/test_block_int8.py"), ["native_per_token_group_quant_int8"], ns)
    out = {}
    for name, dtype in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        torch.manual_seed(13)
        x = (torch.randn(19, 512) * torch.where(torch.rand(19, 512) < 1e-2, 50.0, 1.0)).to(dtype)
        for group in (64, 128):
            q, s = ns["native_per_token_group_quant_int8"](x, group)
            out.update({f"{name}_g{group}_q": q.numpy(), f"{name}_g{group}_s": s.numpy()})
        out[f"{name}_x"] = _np(x)
    np.savez_compressed(os.path.join(HERE, "quant_int8_native.npz"), **out)


def main(reference: str, only: str = ""):
    if only in ("", "int8"):
        make_int8(reference)
        if only:
            print("golden vectors written to", HERE)
            return
    if only in ("", "rmsnorm"):
        make_rmsnorm(reference)
        if only:
            print("golden vectors written to", HERE)
            return
    if only in ("", "ue8m0"):
        make_ue8m0(reference)
        if only:
            print("golden vectors written to", HERE)
            return
    ns = {"torch": torch, "Optional": Optional, "Tuple": Tuple, "Type": Type, "SiluAndMul": _SiluAndMul}
    _extract(os.path.join(reference, "python/sglang/test/test_block_fp8.py"),
             ["native_per_token_group_quant_fp8", "native_w8a8_block_fp8_matmul", "torch_w8a8_block_fp8_moe"], ns)
    _extract(os.path.join(reference, "sgl-kernel/tests/test_fp8_blockwise_gemm.py"), ["baseline_scaled_mm"], ns)
    _extract(os.path.join(reference, "sgl-kernel/tests/test_fp8_blockwise_moe.py"),
             ["calc_diff", "ceil_div", "per_token_cast_to_fp8", "per_block_cast_to_fp8"], ns)
    ka = {"torch": torch}
    _extract(os.path.join(reference, "test/srt/quant/test_fp8_kernel.py"), ["_make_A", "_make_B"], ka,
             inside_class="TestFP8Base")

    # ---------------- quant: reference torch twin on its own test distribution (torch.rand, seed 0)
    out = {}
    for name, dtype in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        torch.manual_seed(0)
        x = torch.rand(7, 512, dtype=dtype)
        q, s = ns["native_per_token_group_quant_fp8"](x, 128)
        out[f"rand_{name}_x"] = _np(x); out[f"rand_{name}_q"] = _np(q); out[f"rand_{name}_s"] = _np(s)
    torch.manual_seed(1)
    x = (torch.randn(83, 1024) * torch.where(torch.rand(83, 1024) < 1e-2, 100.0, 1.0)).to(torch.bfloat16)
    q, s = ns["native_per_token_group_quant_fp8"](x, 128)
    out["randn_bf16_x"] = _np(x); out["randn_bf16_q"] = _np(q); out["randn_bf16_s"] = _np(s)
    np.savez_compressed(os.path.join(HERE, "quant_native.npz"), **out)

    # ---------------- quant: known-answer generator of test_fp8_kernel.py (device kw patched to cpu)
    _rand, _randn = torch.rand, torch.randn
    torch.rand = lambda *a, **k: _rand(*a, **{**k, "device": "cpu"})
    try:
        torch.manual_seed(0)
        A, A_q, A_s = ka["_make_A"](64, 512, 128, FP8)
        B, B_q, B_s = ka["_make_B"](512, 256 + 64, 128, FP8)
    finally:
        torch.rand = _rand
    np.savez_compressed(os.path.join(HERE, "known_answer.npz"),
                        A=_np(A), A_q=_np(A_q), A_s=_np(A_s), B=_np(B), B_q=_np(B_q), B_s=_np(B_s))

    # ---------------- matmul: reference native matmul + sgl-kernel baseline on the same inputs
    torch.manual_seed(0)
    M, N, K = 33, 384, 512
    a = ((torch.rand(M, K) - 0.5) * 2 * 448).to(FP8)
    b = ((torch.rand(N, K) - 0.5) * 2 * 448).to(FP8)
    As = torch.rand(M, K // 128) * 1e-2
    Bs = torch.rand(N // 128, K // 128) * 1e-2
    c32 = ns["native_w8a8_block_fp8_matmul"](a, b, As, Bs, [128, 128], torch.float32)
    cbf = ns["native_w8a8_block_fp8_matmul"](a, b, As, Bs, [128, 128], torch.bfloat16)
    base = ns["baseline_scaled_mm"](a, b.t(), As, Bs.t(), torch.bfloat16)
    np.savez_compressed(os.path.join(HERE, "matmul_native.npz"), a=_np(a), b=_np(b), As=_np(As), Bs=_np(Bs),
                        c_f32=_np(c32), c_bf16=_np(cbf), baseline_bf16=_np(base))

    # ---------------- weight / token casts
    torch.manual_seed(2)
    w = torch.randn(200, 384) * 0.02
    wq, ws = ns["per_block_cast_to_fp8"](w)
    t = torch.randn(5, 256)
    tq, ts = ns["per_token_cast_to_fp8"](t)
    d = ns["calc_diff"](torch.randn(64, 64, generator=torch.Generator().manual_seed(3)),
                        torch.randn(64, 64, generator=torch.Generator().manual_seed(4)))
    np.savez_compressed(os.path.join(HERE, "casts.npz"), w=_np(w), wq=_np(wq), ws=_np(ws),
                        t=_np(t), tq=_np(tq), ts=_np(ts), calc_diff=np.float64(d))

    # ---------------- MoE: reference torch_w8a8_block_fp8_moe
    torch.manual_seed(5)
    Mt, D, I, E, topk = 17, 256, 128, 4, 2
    a = (torch.randn(Mt, D) / 10).to(torch.bfloat16)
    w1 = torch.randn(E, 2 * I, D) * 0.05
    w2 = torch.randn(E, D, I) * 0.05
    w1q, w1s, w2q, w2s = [], [], [], []
    for e in range(E):
        q_, s_ = ns["per_block_cast_to_fp8"](w1[e]); w1q.append(q_); w1s.append(s_)
        q_, s_ = ns["per_block_cast_to_fp8"](w2[e]); w2q.append(q_); w2s.append(s_)
    w1q, w1s, w2q, w2s = torch.stack(w1q), torch.stack(w1s), torch.stack(w2q), torch.stack(w2s)
    score = torch.randn(Mt, E)
    o = ns["torch_w8a8_block_fp8_moe"](a, w1q, w2q, w1s, w2s, score, topk, [128, 128])
    np.savez_compressed(os.path.join(HERE, "moe_native.npz"), a=_np(a), w1q=_np(w1q), w1s=_np(w1s),
                        w2q=_np(w2q), w2s=_np(w2s), score=_np(score), topk=np.int64(topk), out=_np(o))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--only", default="", choices=["", "ue8m0", "rmsnorm", "int8"], help="write just this group of vectors")
    a = ap.parse_args()
    main(a.reference, a.only)

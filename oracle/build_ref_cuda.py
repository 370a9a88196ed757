"""TEST/BENCH INFRASTRUCTURE ONLY -- builds the on-box comparator, never the product.

Compiles the reference's own Blackwell CUDA kernels of the block-FP8 linear path for sm_100a,
from the reference checkout where the sources lie (no source is copied):

    sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu   (CUTLASS sm100 blockwise GEMM)
    sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu  (group quantisation)
    sgl-kernel/csrc/moe/fp8_blockwise_moe_kernel.cu     (CUTLASS sm100 grouped GEMM)
    sgl-kernel/csrc/moe/prepare_moe_input.cu            (routing tables, row shuffles)

plus oracle/ref_cuda_shim.cpp, into three libraries under baseline/_ref/ (one per kernel family,
so that one family that fails to build does not take the others with it):

    baseline/_ref/libsgl_kernel_ref_gemm.so, ..._quant.so, ..._moe.so

The flags mirror sgl-kernel/CMakeLists.txt:137-192 (no -use_fast_math).  CUTLASS and FlashInfer
headers come from the flashinfer package in site-packages: a CUTLASS 4.x tree, not the commit the
reference pins (the pinned trees are not part of the reference checkout).  nvcc cross-compiles
without a GPU; each CUTLASS translation unit takes 8-10 minutes.

Usage:  python oracle/build_ref_cuda.py [--reference /path/to/reference] [--only gemm,quant,moe] [--force]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
import time
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(os.path.dirname(HERE), "baseline", "_ref")
OBJ_DIR = os.path.join(HERE, "_build")
SHIM = os.path.join(HERE, "ref_cuda_shim.cpp")

FAMILIES = {
    "gemm": (["csrc/gemm/fp8_blockwise_gemm_kernel.cu"], "REF_SHIM_GEMM"),
    "quant": (["csrc/gemm/per_token_group_quant_8bit.cu"], "REF_SHIM_QUANT"),
    "moe": (["csrc/moe/fp8_blockwise_moe_kernel.cu", "csrc/moe/prepare_moe_input.cu"], "REF_SHIM_MOE"),
}


def lib_path(family: str) -> str:
    return os.path.join(OUT_DIR, f"libsgl_kernel_ref_{family}.so")


def _site_packages() -> str:
    import flashinfer

    return os.path.dirname(os.path.dirname(os.path.abspath(flashinfer.__file__)))


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.isfile(cand) else "nvcc"


def _flags(reference: str):
    import torch
    from torch.utils import cpp_extension

    sp = _site_packages()
    sk = os.path.join(reference, "sgl-kernel")
    inc = cpp_extension.include_paths() + [
        sysconfig.get_paths()["include"],
        os.path.join(sk, "include"), os.path.join(sk, "csrc"), os.path.join(sk, "csrc", "moe"),
        os.path.join(sp, "flashinfer", "data", "include"),
        os.path.join(sp, "flashinfer", "data", "cutlass", "include"),
        os.path.join(sp, "flashinfer", "data", "cutlass", "tools", "util", "include"),
    ]
    flags = ["-std=c++17", "-O3", "-gencode=arch=compute_100a,code=sm_100a", "-DNDEBUG",
             "-DCUTE_USE_PACKED_TUPLE=1", "-DCUTLASS_ENABLE_TENSOR_CORE_MMA=1",
             "-DCUTLASS_VERSIONS_GENERATED", "-DCUTLASS_TEST_LEVEL=0", "-DCUTLASS_TEST_ENABLE_CACHED_RESULTS=1",
             "-DCUTLASS_DEBUG_TRACE_LEVEL=0",
             "-DFLASHINFER_ENABLE_F16", "-DFLASHINFER_ENABLE_BF16", "-DFLASHINFER_ENABLE_FP8",
             "-DFLASHINFER_ENABLE_FP8_E4M3", "-DFLASHINFER_ENABLE_FP8_E5M2",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
             "--expt-relaxed-constexpr", "--expt-extended-lambda", "-w", "-Xcompiler", "-fPIC"]
    return flags + [f"-I{p}" for p in inc]


def build(reference: str, only=None, force: bool = False, verbose: bool = True) -> dict:
    """Build the requested families; returns {family: path or None}."""
    import torch

    sk = os.path.join(reference, "sgl-kernel")
    fams = [f for f in FAMILIES if only is None or f in only]
    out = {}
    if not os.path.isdir(sk):
        for f in fams:
            out[f] = lib_path(f) if os.path.isfile(lib_path(f)) else None
        return out
    os.makedirs(OUT_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    flags = _flags(reference)
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")

    def one(family: str):
        srcs, macro = FAMILIES[family]
        srcs = [os.path.join(sk, s) for s in srcs]
        target = lib_path(family)
        if os.path.isfile(target) and not force:
            if os.path.getmtime(target) >= max(os.path.getmtime(p) for p in srcs + [SHIM, __file__]):
                return family, target
        objs = []
        t0 = time.time()
        for s in srcs + [SHIM]:
            obj = os.path.join(OBJ_DIR, f"ref_{family}_{os.path.basename(s).rsplit('.', 1)[0]}.o")
            cmd = [_nvcc()] + flags + [f"-D{macro}", "-x", "cu", "-c", s, "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            with open(obj[:-2] + ".log", "w") as f:
                f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                if verbose:
                    print(f"[build_ref_cuda] {family}: nvcc failed for {s} (log {obj[:-2]}.log)")
                return family, None
            objs.append(obj)
        cmd = [_nvcc(), "-shared", "-o", target] + objs + [f"-L{torch_lib}", f"-Xlinker", f"-rpath={torch_lib}",
                                                           "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10",
                                                           "-lc10_cuda", "-lcuda", "-cudart", "shared"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            if verbose:
                print(f"[build_ref_cuda] {family}: link failed:\n{r.stderr}")
            return family, None
        if verbose:
            print(f"[build_ref_cuda] {family}: built {target} in {time.time() - t0:.0f} s")
        return family, target

    with ThreadPoolExecutor(max_workers=len(fams) or 1) as ex:
        for fam, path in ex.map(one, fams):
            out[fam] = path
    return out


def load(family: str) -> bool:
    """Load one built family into torch (registers torch.ops.sgl_kernel_ref.*); False when absent."""
    p = lib_path(family)
    if not os.path.isfile(p):
        return False
    import torch

    torch.ops.load_library(p)
    return True


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("SGLANG_REFERENCE_DIR"),
                    help="path of the reference checkout (or set SGLANG_REFERENCE_DIR)")
    ap.add_argument("--only", default=None, help="comma-separated subset of gemm,quant,moe")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    if not a.reference:
        ap.error("--reference or SGLANG_REFERENCE_DIR is required")
    res = build(a.reference, a.only.split(",") if a.only else None, a.force)
    print("[build_ref_cuda] ->", res)
    sys.exit(0)

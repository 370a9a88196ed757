"""TEST/BENCH INFRASTRUCTURE ONLY -- builds the checker, never the product.

Compiles the reference's own CPU block-FP8 matmul from the reference checkout
(sgl-kernel/csrc/cpu/gemm.cpp and gemm_fp8.cpp, compiled where they lie; no
source is copied) plus oracle/ref_cpu_shim.cpp into
oracle/_ref/libsgl_kernel_ref_cpu.so.

The reference kernels need AVX512F + AVX512-BF16 + AMX-BF16 at compile time
(sgl-kernel/csrc/cpu/vec.h:3-5); without them every kernel body is a
"scalar path not implemented" check, so the build is skipped when the host
lacks those flags.  The flags mirror sgl-kernel/csrc/cpu/CMakeLists.txt
(-O3 -fopenmp -march=native, SGLANG_CPU_FP8_CVT_FTZ default ON).

Usage:  python oracle/build_ref.py [--reference /path/to/reference] [--force]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT_SO = os.path.join(OUT_DIR, "libsgl_kernel_ref_cpu.so")
NEEDED_CPU_FLAGS = ("avx512f", "avx512_bf16", "amx_bf16", "amx_tile")


def host_has_amx() -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = set(line.split(":", 1)[1].split())
                    return all(x in flags for x in NEEDED_CPU_FLAGS)
    except OSError:
        pass
    return False


def build(reference: str, force: bool = False, verbose: bool = True) -> str | None:
    """Return the path of the built library, or None when it cannot be built here."""
    src_dir = os.path.join(reference, "sgl-kernel", "csrc", "cpu")
    srcs = [os.path.join(src_dir, "gemm.cpp"), os.path.join(src_dir, "gemm_fp8.cpp")]
    if not all(os.path.isfile(s) for s in srcs):
        if verbose:
            print(f"[build_ref] reference sources not found under {reference}; skipped")
        return OUT_SO if os.path.isfile(OUT_SO) else None
    if not host_has_amx():
        if verbose:
            print("[build_ref] host lacks AVX512-BF16/AMX; reference CPU op not buildable here")
        return None
    shim = os.path.join(HERE, "ref_cpu_shim.cpp")
    if os.path.isfile(OUT_SO) and not force:
        newest = max(os.path.getmtime(p) for p in srcs + [shim, __file__])
        if os.path.getmtime(OUT_SO) >= newest:
            return OUT_SO
    import torch
    from torch.utils import cpp_extension

    os.makedirs(OUT_DIR, exist_ok=True)
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    inc = cpp_extension.include_paths() + [
        sysconfig.get_paths()["include"],
        os.path.join(reference, "sgl-kernel", "csrc"),
        os.path.join(reference, "sgl-kernel", "include"),
        src_dir,
    ]
    cmd = ["g++", "-O3", "-std=c++17", "-march=native", "-fopenmp", "-fPIC", "-shared", "-w",
           "-DSGLANG_CPU_FP8_CVT_FTZ",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{p}" for p in inc]
    cmd += srcs + [shim, "-o", OUT_SO, f"-L{torch_lib}", f"-Wl,-rpath,{torch_lib}",
                   "-ltorch", "-ltorch_cpu", "-lc10"]
    if verbose:
        print("[build_ref]", " ".join(cmd))
    subprocess.check_call(cmd)
    return OUT_SO


def load() -> bool:
    """Load the built library into torch (registers torch.ops.sgl_kernel_ref.*)."""
    if not os.path.isfile(OUT_SO) or not host_has_amx():
        return False
    import torch

    torch.ops.load_library(OUT_SO)
    return True


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("SGLANG_REFERENCE_DIR"),
                    help="path of the reference checkout (or set SGLANG_REFERENCE_DIR)")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    if not a.reference:
        ap.error("--reference or SGLANG_REFERENCE_DIR is required")
    out = build(a.reference, a.force)
    print("[build_ref] ->", out)
    sys.exit(0)

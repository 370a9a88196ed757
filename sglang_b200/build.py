"""Builds libb200_block_fp8.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m sglang_b200.build [--force] [--verbose]

The library has no torch dependency; it links only the CUDA runtime.  Object files go to
sglang_b200/csrc/_build/, the shared library next to this file.
"""
from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "_build")
LIB = os.path.join(PKG, "libb200_block_fp8.so")
HEADER = os.path.join(os.path.dirname(PKG), "include", "b200_block_fp8.h")

NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.isfile(cand) else "nvcc"


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime() -> float:
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + [HEADER, __file__]
    return max(os.path.getmtime(h) for h in hdrs)


# Kernels that move registers between warpgroups with setmaxnreg: the arithmetic in their Cfg structs
# assumes the launch allocates exactly this many registers per thread.  If ptxas ever allocates fewer,
# setmaxnreg.inc would wait for registers nobody releases, so the build refuses the object instead.
_FIXED_REGS = [
    (re.compile(r"gemm_block_fp8_kernelILi(128|256)ELi16E"), 96),
    (re.compile(r"gemm_block_fp8_swapab_kernelILi128E"), 168),
]


def check_register_counts(ptxas_log: str) -> None:
    name = None
    for line in ptxas_log.splitlines():
        m = re.search(r"Compiling entry function '([^']+)'", line)
        if m:
            name = m.group(1)
            continue
        m = re.search(r"Used (\d+) registers", line)
        if m and name:
            for pat, want in _FIXED_REGS:
                if pat.search(name) and int(m.group(1)) != want:
                    raise RuntimeError(f"{name}: ptxas allocated {m.group(1)} registers, the kernel's register "
                                       f"rebalancing needs {want}")
            name = None


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    dep_t = _deps_mtime()
    jobs = []
    for src in sources():
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if force or not os.path.isfile(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), dep_t):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [_nvcc()] + NVCC_FLAGS + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        with open(obj[:-2] + ".ptxas.log", "w") as f:
            f.write(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stderr}")
        try:
            check_register_counts(r.stderr)
        except RuntimeError:
            os.remove(obj)
            raise
        if verbose:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    objs = [os.path.join(OBJ, os.path.basename(s)[:-3] + ".o") for s in sources()]
    if jobs or force or not os.path.isfile(LIB):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-cudart", "shared"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)

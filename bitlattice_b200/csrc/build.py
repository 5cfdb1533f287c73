"""Builds libbitlattice_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python bitlattice_b200/csrc/build.py [--force] [--verbose]

The kernels that must reproduce the reference's fp32 rounding bit for bit (update.cu, quant.cu, swiglu.cu) are compiled with
--fmad=false, as the reference's extension is (its setup.py:21-22); the GEMM keeps fused multiply-adds.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB = os.path.join(PKG, "libbitlattice_b200.so")
OBJ = os.path.join(HERE, "_build")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden",
          "-Xptxas", "-v"]
SOURCES = {
    "abi.cu": [],
    "update.cu": ["--fmad=false"],
    "quant.cu": ["--fmad=false"],
    "quant_general.cu": ["--fmad=false"],
    "gemm.cu": [],
    "swiglu.cu": ["--fmad=false"],
    "gather.cu": [],
}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(PKG), "include", "bitlattice_b200.h"))
    objs = []
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    for src, extra in SOURCES.items():
        path = os.path.join(HERE, src)
        if not os.path.exists(path):
            continue
        obj = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [path] + headers):
            cmd = [_nvcc(), *ARCH, *COMMON, *extra, "-c", path, "-o", obj]
            res = subprocess.run(cmd, capture_output=True, text=True, env=env)
            log = os.path.join(OBJ, src + ".log")
            with open(log, "w") as f:
                f.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
            if verbose or res.returncode:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode:
                raise RuntimeError(f"nvcc failed on {src} (log: {log})")
    if force or _stale(LIB, objs):
        cmd = [_nvcc(), *ARCH, "-shared", "-o", LIB, *objs, "-cudart", "static"]
        res = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("linking libbitlattice_b200.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

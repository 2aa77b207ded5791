"""Build the CUDA library in-tree: oxmera_b200/liboxmera_b200.so.

`python -m oxmera_b200.build [--force] [-v]`.  nvcc cross-compiles for sm_100a
without a GPU.  The translation units compile in parallel and are linked into
one shared library; a Rust build.rs would run the same command lines.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
# the longest units first: they decide the wall time of a parallel build
SOURCES = ["gemm_f16_kk.cu", "gemm_f16_kn.cu", "gemm_f16_mk.cu", "gemm_f16_mn.cu", "gemm_f8_kk.cu", "gemm_f8_kn.cu", "gemm_f8_mk.cu",
           "gemm_f8_mn.cu", "gemm_tf32.cu", "api.cu", "gemm_mx.cu"]
OUT = os.path.join(HERE, "liboxmera_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]


def compile_command(src: str, verbose: bool = False):
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    return ["nvcc", *NVCC_FLAGS, *(("-Xptxas", "-v") if verbose else ()), "-c", os.path.join(CSRC, src), "-o", obj], obj


def link_command(objs):
    return ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", OUT, *objs]


def is_stale() -> bool:
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    deps = glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        [os.path.join(HERE, "..", "include", "oxmera_b200.h")]
    return any(os.path.getmtime(d) > built for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile when the library is missing or older than its sources."""
    if not force and not is_stale():
        return OUT
    os.makedirs(OBJ, exist_ok=True)

    def run(src):
        cmd, obj = compile_command(src, verbose)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed ({res.returncode}):\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        return obj

    # a translation unit is recompiled when its object is older than the unit itself or any header
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(HERE, "..", "include", "oxmera_b200.h")]
    newest_header = max(os.path.getmtime(h) for h in headers)

    def fresh(src):
        obj = compile_command(src)[1]
        return (not force and os.path.exists(obj) and
                os.path.getmtime(obj) >= max(newest_header, os.path.getmtime(os.path.join(CSRC, src))))

    todo = [s for s in SOURCES if not fresh(s)]
    with ThreadPoolExecutor(max_workers=min(max(len(todo), 1), os.cpu_count() or 1)) as pool:
        list(pool.map(run, todo))
    objs = [compile_command(s)[1] for s in SOURCES]
    res = subprocess.run(link_command(objs), capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return OUT


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))

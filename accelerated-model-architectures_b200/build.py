"""Builds libxma_b200.so (all CUDA kernels + the C ABI) in-tree with nvcc for sm_100a.

Run as a script (`python build.py [--force]`) or call `build()`; the library lands in
`xma/lib/libxma_b200.so` next to the Python host layer that loads it with ctypes. nvcc
cross-compiles, so no GPU is needed to build.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_DIR = os.path.join(_HERE, "xma", "lib")
LIB_PATH = os.path.join(LIB_DIR, "libxma_b200.so")
OBJ_DIR = os.path.join(_HERE, "build")

SOURCES = ["routing.cu", "permute.cu", "swiglu.cu", "gemm_simt.cu", "grouped_gemm_sm100.cu", "grouped_gemm_sm100_2cta.cu",
           "gemm_api.cu", "expert_parallel.cu", "rmsnorm.cu", "aux_loss.cu", "sequence_packing.cu"]
HEADERS = ["common.cuh", "gemm_internal.h", "sm100_common.cuh"]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; cannot build libxma_b200.so")
    return exe


def _newest_source_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return max(os.path.getmtime(p) for p in paths)


def is_up_to_date() -> bool:
    return os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _newest_source_mtime()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and is_up_to_date():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, SOURCES))

    tmp = LIB_PATH + ".tmp"
    res = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
                         capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)

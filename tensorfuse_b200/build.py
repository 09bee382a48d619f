"""Compile libtensorfuse.so (sm_100a only) in-tree with nvcc.

    python tensorfuse_b200/build.py [--force]

The shared library lands in tensorfuse_b200/lib/ and is what both the ctypes
layer of this package and a C/C++ caller link against.  nvcc cross-compiles, so
this works on a machine without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "build")
LIB = os.path.join(LIBDIR, "libtensorfuse.so")

SOURCES = ["softmax_dropout.cu", "gemm_simt.cu", "gemm_tc.cu", "attention.cu", "quantize.cu", "layernorm.cu", "transformer_layer.cpp", "runtime.cpp", "c_api.cpp",
           "host_ops.cpp", "noalloc.cu", "profiler.cpp", "cxx_api.cpp"]
HEADERS = ["kernels.h", "ptx.cuh", "epilogue.cuh", "runtime.h", "gemm_tc_kernel.cuh", "gemm_tc_pair_kernel.cuh", "gemm_tf32x3_kernel.cuh", "attention_tc_kernel.cuh", "philox.cuh", "tma_host.h"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=default", "-DTENSORFUSE_WITH_CUDA_RUNTIME",
              "-I", os.path.join(ROOT, "include"), "-I", CSRC]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libtensorfuse.so cannot be built")
    return exe


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    deps += [os.path.join(ROOT, "include", "tensorfuse_b200.h"), os.path.join(ROOT, "include", "tensorfuse.h")]
    deps += [os.path.join(ROOT, "include", "tensorfuse", f) for f in ("types.h", "tensorfuse.h", "kernels.h", "profiler.h")]
    return _newest(deps) > os.path.getmtime(LIB)


def _compile(src: str) -> str:
    obj = os.path.join(OBJDIR, os.path.splitext(src)[0] + ".o")
    cmd = [nvcc(), *NVCC_FLAGS, "-x", "cu", "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    with cf.ThreadPoolExecutor(max_workers=min(6, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(_compile, SOURCES))
    cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print("built", LIB)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)

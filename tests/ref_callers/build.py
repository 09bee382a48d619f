"""Build the reference's own callers, unmodified, against libtensorfuse.so.

    python tests/ref_callers/build.py /path/to/TensorFuse-checkout

The reference ships test programs, a benchmark and Python tests that exercise
its library through the C interface, the flat wrappers, the mangled C++
symbols and the `tensorfuse` Python package.  This script copies them from a
checkout of the reference into the git-ignored directory baseline/_ref/ref_callers/,
compiles every program exactly as it is (nvcc, sm_100a) and links it against
THIS repository's library.  No source file is edited; the one relative
include of the reference's headers (`#include "../tensorfuse/types.h"` in
test_c_api_debug.cpp) is satisfied by a copy of this repository's
include/tensorfuse/ placed where that path points.

It also compiles the reference's own GPU library for sm_100a, from its sources
where they lie in the checkout, into baseline/_ref/ref_lib/: the kernels this
repository replaces, as a second comparator on a GPU (tests/test_reference_library_gpu.py,
and the `reference_gpu_kernels` leg of bench.py).  That library needs NVIDIA
CUTLASS headers, which the reference does not vendor; the recipe takes them from
$CUTLASS_INCLUDE or from a Python package that ships them, and skips the step
(recording why in the manifest) when there are none.

Outputs (all under baseline/_ref/, none of it version controlled):
    ref_lib/libtensorfuse_reference.so   the reference's library (optional, see above)
  and under ref_callers/:
    bin/<program>               executables, rpath -> tensorfuse_b200/lib
    py/tensorfuse/*.py          the reference's pure-Python package, verbatim, plus a
                                two-line _tensorfuse.py that re-exports this
                                repository's binding module in place of the pybind one
    py/tests/*.py               the reference's Python tests, verbatim
    manifest.json               what was built, with the source path of every file

tests/test_ref_callers_gpu.py runs the results on a GPU.
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(ROOT, "baseline", "_ref", "ref_callers")
LIBDIR = os.path.join(ROOT, "tensorfuse_b200", "lib")

# (source path inside the reference, extra link flags)
PROGRAMS = [
    ("src/tests/test_c_api_debug.cpp", []),
    ("src/tests/test_wrapper_debug.cpp", []),
    ("src/tests/test_kernels_simple.cpp", ["-ldl"]),
    ("src/tests/test_working_kernel.cu", ["-ldl"]),
    ("src/tests/test_kernels.cu", []),
    ("src/tests/test_gemm_edge_cases.cu", []),
    ("src/tests/test_softmax_dropout.cu", []),
    ("benchmarks/bert_baseline.cu", ["-lcublas", "-lcublasLt"]),
]
HEADERS = ["benchmarks/tensorfuse_c_api.h"]
PY_PACKAGE = ["__init__.py", "core.py", "memory.py", "profiler.py", "utils.py"]
PY_TESTS = ["test_mathematical_verification.py", "test_int8_tensor_cores.py", "test_core_bindings.py",
            "test_numpy_integration.py"]

SHIM = '''"""Stands where the reference's compiled pybind11 module sits
(src/python/tensorfuse_python.cpp:26); re-exports this repository's binding."""
from tensorfuse_b200._tensorfuse import *  # noqa: F401,F403
from tensorfuse_b200._tensorfuse import (Status, DataType, Layout, Shape, Config, Tensor,  # noqa: F401
                                         ProfileConfig, Metrics, RooflineModel)
'''


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


REF_LIB_DIR = os.path.join(ROOT, "baseline", "_ref", "ref_lib")
REF_LIB = os.path.join(REF_LIB_DIR, "libtensorfuse_reference.so")
REF_LIB_SOURCES = ["src/tensorfuse_c_api.cpp", "src/utils/error_handling.cpp", "src/kernels/fused_gemm_bias_gelu.cu",
                   "src/kernels/fused_gemm_bias_gelu_int8.cu", "src/kernels/fused_gemm_bias_gelu_optimized.cu",
                   "src/kernels/fused_softmax_dropout.cu"]


def cutlass_include() -> str | None:
    """A CUTLASS header tree: $CUTLASS_INCLUDE, else one shipped inside a Python package."""
    env = os.environ.get("CUTLASS_INCLUDE")
    if env and os.path.isdir(os.path.join(env, "cutlass")):
        return env
    import importlib.util
    for pkg, rel in (("flashinfer", "data/cutlass/include"), ("tilelang", "3rdparty/cutlass/include")):
        spec = importlib.util.find_spec(pkg)
        if spec and spec.origin:
            cand = os.path.join(os.path.dirname(spec.origin), rel)
            if os.path.isdir(os.path.join(cand, "cutlass")):
                return cand
    return None


def build_reference_library(reference: str, verbose: bool = True) -> dict:
    """The reference's C API + kernels, compiled for sm_100a as they are (nothing is
    copied or edited; only the shared library lands in baseline/_ref/ref_lib/)."""
    info = {"ok": False, "path": REF_LIB, "sources": REF_LIB_SOURCES}
    inc = cutlass_include()
    if inc is None:
        info["skipped"] = "no CUTLASS headers (set CUTLASS_INCLUDE)"
        return info
    os.makedirs(REF_LIB_DIR, exist_ok=True)
    srcs = [os.path.join(reference, f) for f in REF_LIB_SOURCES]
    if os.path.exists(REF_LIB) and all(os.path.getmtime(REF_LIB) > os.path.getmtime(f) for f in srcs):
        info["ok"] = True
        info["cached"] = True
        return info
    cmd = [nvcc(), "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr",
           "--expt-extended-lambda", "--use_fast_math", "-O3", "-w", "-Xcompiler", "-fPIC", "-shared",
           "-I", os.path.join(reference, "src"), "-I", inc, "-o", REF_LIB, *srcs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    info["ok"] = r.returncode == 0
    info["cutlass_include"] = inc
    if r.returncode:
        info["log"] = (r.stdout + r.stderr)[-2000:]
    if verbose:
        print(("built  " if info["ok"] else "FAILED ") + "the reference's GPU library -> " + REF_LIB)
    return info


def build(reference: str, verbose: bool = True) -> dict:
    if not os.path.isdir(os.path.join(reference, "src", "tests")):
        raise RuntimeError(f"{reference} is not a checkout of the reference")
    if not os.path.exists(os.path.join(LIBDIR, "libtensorfuse.so")):
        raise RuntimeError("build tensorfuse_b200/lib/libtensorfuse.so first (python tensorfuse_b200/build.py)")
    if os.path.isdir(OUT):
        shutil.rmtree(OUT)
    bindir = os.path.join(OUT, "bin")
    os.makedirs(bindir)
    manifest = {"reference": reference, "programs": {}, "python": {}}

    # sources keep their relative places so that relative includes resolve
    for rel, _ in PROGRAMS:
        dst = os.path.join(OUT, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(reference, rel), dst)
    for rel in HEADERS:
        dst = os.path.join(OUT, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(reference, rel), dst)
    # "../tensorfuse/types.h" seen from src/tests/ -> this repository's headers
    shutil.copytree(os.path.join(ROOT, "include", "tensorfuse"), os.path.join(OUT, "src", "tensorfuse"))

    for rel, extra in PROGRAMS:
        name = os.path.splitext(os.path.basename(rel))[0]
        exe = os.path.join(bindir, name)
        cmd = [nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-w", "-x", "cu",
               os.path.join(OUT, rel), "-o", exe, "-I", os.path.join(ROOT, "include"), "-L", LIBDIR, "-ltensorfuse",
               "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../../tensorfuse_b200/lib", *extra]
        r = subprocess.run(cmd, capture_output=True, text=True)
        manifest["programs"][name] = {"source": rel, "ok": r.returncode == 0,
                                      "log": (r.stdout + r.stderr)[-2000:] if r.returncode else ""}
        if verbose:
            print(("built  " if r.returncode == 0 else "FAILED ") + rel)
            if r.returncode:
                print(r.stdout + r.stderr)

    pkg = os.path.join(OUT, "py", "tensorfuse")
    os.makedirs(pkg)
    for f in PY_PACKAGE:
        shutil.copyfile(os.path.join(reference, "src", "python", "tensorfuse", f), os.path.join(pkg, f))
        manifest["python"][f"tensorfuse/{f}"] = f"src/python/tensorfuse/{f}"
    with open(os.path.join(pkg, "_tensorfuse.py"), "w") as fh:
        fh.write(SHIM)
    tests = os.path.join(OUT, "py", "tests")
    os.makedirs(tests)
    for f in PY_TESTS:
        shutil.copyfile(os.path.join(reference, "src", "tests", "python", f), os.path.join(tests, f))
        manifest["python"][f"tests/{f}"] = f"src/tests/python/{f}"
    manifest["reference_library"] = build_reference_library(reference, verbose)
    with open(os.path.join(OUT, "manifest.json"), "w") as fh:
        json.dump(manifest, fh, indent=1)
    failed = [n for n, v in manifest["programs"].items() if not v["ok"]]
    if failed:
        raise RuntimeError("reference callers that did not compile/link: " + ", ".join(failed))
    return manifest


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TENSORFUSE_REFERENCE", "")
    if not ref:
        sys.exit("usage: build.py <checkout of the reference>  (or set TENSORFUSE_REFERENCE)")
    build(ref)
    print("reference callers built under", OUT)

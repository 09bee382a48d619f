"""The reference's own callers, unmodified, running on libtensorfuse.so.

tests/ref_callers/build.py compiles the reference's C++/CUDA test programs and
its benchmark against this library and stages the reference's pure-Python
package over this repository's `_tensorfuse` module.  Here every artefact is
run on the GPU: exit status 0 and no failure marker in the output is the bar
(several of the programs print FAILED and still return 0, so the text is
checked as well).  Nothing in these programs was written for this repository:
they are the reference's statement of what a caller expects of the library
(reference src/tests/*.cpp|*.cu, src/tests/python/*.py, benchmarks/bert_baseline.cu).
"""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OUT = os.path.join(ROOT, "baseline", "_ref", "ref_callers")
BIN = os.path.join(OUT, "bin")
LIBDIR = os.path.join(ROOT, "tensorfuse_b200", "lib")

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.isdir(BIN),
                                 reason="reference callers not built (python tests/ref_callers/build.py <reference>)")]

FAIL_MARKS = ("FAILED", "FAILURE", "FAIL!", "❌")

# name -> reference file and what it checks
PROGRAMS = {
    "test_c_api_debug": "struct C interface, 1x1x1 FP32: GELU(2.5) within 1e-4 (src/tests/test_c_api_debug.cpp:94-170)",
    "test_wrapper_debug": "flat fp32 wrapper, same known answer (src/tests/test_wrapper_debug.cpp:16-114)",
    "test_kernels_simple": "dlopen + dlsym of the mangled fp32/fp16 launchers (src/tests/test_kernels_simple.cpp:62-63)",
    "test_working_kernel": "dlsym'd fp32 launcher on 8x16x32 all-0.1 inputs (src/tests/test_working_kernel.cu:75-135)",
    "test_kernels": "FP32 64x128x256 vs the CPU loop at 1e-4, FP16 runs (src/tests/test_kernels.cu:43-194)",
    "test_gemm_edge_cases": "size / alpha-beta / extreme-value grids at 1e-4 / 1e-2 (src/tests/test_gemm_edge_cases.cu:78-383)",
    "test_softmax_dropout": "row sums, non-negativity, keep rate at p = 0.1 (src/tests/test_softmax_dropout.cu:108-337)",
}


def _run(cmd, cwd, env=None, timeout=600):
    r = subprocess.run(cmd, cwd=cwd, env=env, capture_output=True, text=True, timeout=timeout)
    return r.returncode, r.stdout + r.stderr


@pytest.mark.parametrize("name", sorted(PROGRAMS))
def test_reference_program(name):
    exe = os.path.join(BIN, name)
    assert os.path.exists(exe), f"{name} was not built"
    # the dlopen-based programs look for ./libtensorfuse.so
    rc, out = _run([exe], cwd=LIBDIR)
    assert rc == 0, f"{name} ({PROGRAMS[name]}) exited {rc}:\n{out[-3000:]}"
    for mark in FAIL_MARKS:
        assert mark not in out, f"{name} ({PROGRAMS[name]}) reported a failure:\n{out[-3000:]}"


def test_reference_benchmark_links_and_runs(tmp_path):
    """benchmarks/bert_baseline.cu: the FP32 BERT-base FFN layer, cuBLASLt against
    the two fused_gemm_bias_gelu_fp32_wrapper calls, 10 + 100 iterations.  It
    needs tensorfuse_simple_init/_cleanup from the library."""
    exe = os.path.join(BIN, "bert_baseline")
    assert os.path.exists(exe)
    os.makedirs(tmp_path / "benchmarks" / "results")
    rc, out = _run([exe], cwd=str(tmp_path))
    assert rc == 0, out[-3000:]
    res = json.loads((tmp_path / "benchmarks" / "results" / "bert_baseline_results.json").read_text())
    rows = {r["name"]: r for r in res["bert_base_benchmark"]["results"]}
    assert rows["TensorFuse_fused"]["avg_time_ms"] > 0 and rows["cuBLASLt_baseline"]["avg_time_ms"] > 0
    print("reference benchmark on this library:", json.dumps(rows))


def _pyenv():
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([os.path.join(OUT, "py"), ROOT, env.get("PYTHONPATH", "")])
    return env


def test_reference_package_imports_without_stub_fallback():
    """The reference's __init__ falls back to stubs (with a warning) when any of
    ~30 names is missing from _tensorfuse (src/python/tensorfuse/__init__.py:53-95, 393-396)."""
    code = ("import warnings; warnings.simplefilter('error'); import tensorfuse, os; "
            "assert os.path.join('ref_callers', 'py') in tensorfuse.__file__; "
            "tensorfuse.init(); print(tensorfuse.get_device_info()); tensorfuse.shutdown()")
    rc, out = _run([sys.executable, "-c", code], cwd=str(OUT), env=_pyenv())
    assert rc == 0, out[-3000:]


# file -> tests that skip themselves whatever the library does:
#   test_mathematical_verification.py:179 skips its alpha/beta case unconditionally;
#   test_numpy_integration.py:72 skips when numpy has no bfloat16.
# Any other skip means the test gave up on the library ("GPU not available: ...").
PY_TESTS = {"test_mathematical_verification.py": 1, "test_int8_tensor_cores.py": 0,
            "test_core_bindings.py": 0, "test_numpy_integration.py": 1}


@pytest.mark.parametrize("test_file", sorted(PY_TESTS))
def test_reference_python_tests(test_file):
    """The reference's Python tests against the reference's package over this library."""
    import re
    path = os.path.join(OUT, "py", "tests", test_file)
    assert os.path.exists(path)
    rc, out = _run([sys.executable, "-m", "pytest", "-q", "-rs", "-p", "no:cacheprovider", path],
                   cwd=os.path.join(OUT, "py", "tests"), env=_pyenv(), timeout=1200)
    assert rc == 0, out[-6000:]
    summary = out.strip().splitlines()[-1]
    passed = int(re.search(r"(\d+) passed", summary).group(1))
    skipped = int(m.group(1)) if (m := re.search(r"(\d+) skipped", summary)) else 0
    assert passed >= 3 and skipped <= PY_TESTS[test_file] and "failed" not in summary, out[-3000:]

"""This library against the reference's own GPU library on the same inputs.

tests/ref_callers/build.py compiles the reference's C API and kernels for
sm_100a (from a checkout, against CUTLASS headers that the reference does not
vendor) into baseline/_ref/ref_lib/.  tests/ref_callers/run_reference_library.py
runs it in a process of its own; here its outputs are compared with this
library's on the same seeded operands.  This pins the paths the reference's own
tests leave unpinned (FP16: "runs"; INT8: 15 % of the maximum) against what the
reference actually computes on this GPU.

Tolerances.  FP32 GEMM: 1e-4 absolute (reference src/tests/test_kernels.cu:139).
FP16 GEMM: the reference rounds the pre-activation to FP16 before its separate
bias+GELU kernel rounds again (src/kernels/fused_gemm_bias_gelu_optimized.cu:24-55,
192-250); this library rounds once, so the two differ by the reference's extra
rounding: 1e-2 relative + 1e-3 absolute.  INT8 (scaled FP32 convention of
src/kernels/fused_gemm_bias_gelu_int8.cu:51-99): 1e-3 relative to the largest
magnitude (the reference is built with --use_fast_math).  Softmax at p = 0: 1e-4
absolute in FP32 (src/tests/python/test_mathematical_verification.py), two FP16
ulps in FP16.  With dropout the two libraries draw from different generators:
both must keep about 1 - p of the elements and scale the kept ones by 1/(1-p).
"""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "baseline", "_ref", "ref_lib", "libtensorfuse_reference.so")
RUNNER = os.path.join(ROOT, "tests", "ref_callers", "run_reference_library.py")

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.exists(REF_LIB),
                                 reason="the reference's GPU library is not built (python tests/ref_callers/build.py <reference>)")]


def make_cases():
    rng = np.random.default_rng(11)
    c = {}
    for tag, (M, K, N) in {"a": (64, 256, 128), "b": (256, 384, 512)}.items():       # 64x128x256: the reference's own test size
        c[f"gemm_f32_{tag}/A"] = rng.standard_normal((M, K)).astype(np.float32)
        c[f"gemm_f32_{tag}/B"] = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
        c[f"gemm_f32_{tag}/bias"] = (rng.standard_normal(N) * 0.5).astype(np.float32)
    for tag, (M, K, N) in {"a": (256, 256, 512), "b": (1024, 512, 1024)}.items():
        c[f"gemm_f16_{tag}/A"] = rng.standard_normal((M, K)).astype(np.float16)
        c[f"gemm_f16_{tag}/B"] = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16)
        c[f"gemm_f16_{tag}/bias"] = (rng.standard_normal(N) * 0.5).astype(np.float16)
    M, K, N = 256, 256, 512
    x, w = rng.standard_normal((M, K)), rng.standard_normal((K, N)) / np.sqrt(K)
    sA, sB = 127.0 / np.abs(x).max(), 127.0 / np.abs(w).max()           # the reference's convention: q = round(x * scale)
    c["gemm_i8_a/A"] = np.clip(np.rint(x * sA), -127, 127).astype(np.int8)
    c["gemm_i8_a/B"] = np.clip(np.rint(w * sB), -127, 127).astype(np.int8)
    c["gemm_i8_a/bias"] = (rng.standard_normal(N) * 0.1).astype(np.float32)
    c["gemm_i8_a/scales"] = np.array([sA, sB], dtype=np.float32)
    for tag, dt, p in (("f32_p0", np.float32, 0.0), ("f16_p0", np.float16, 0.0), ("f16_p02", np.float16, 0.2)):
        c[f"softmax_{tag}/x"] = (rng.standard_normal((2, 4, 64, 128)) * 2).astype(dt)
        c[f"softmax_{tag}/p"] = np.array([p], dtype=np.float32)
        c[f"softmax_{tag}/seed"] = np.array([5], dtype=np.uint64)
    return c


@pytest.fixture(scope="module")
def reference_outputs(tmp_path_factory):
    d = tmp_path_factory.mktemp("reflib")
    src, dst = str(d / "in.npz"), str(d / "out.npz")
    cases = make_cases()
    np.savez(src, **cases)
    r = subprocess.run([sys.executable, RUNNER, "cases", src, dst], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return cases, np.load(dst)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_fp32_gemm_matches_the_reference_kernels(tf, reference_outputs, tag):
    cases, ref = reference_outputs
    g = f"gemm_f32_{tag}"
    assert int(ref[f"{g}/status"][0]) == 0
    mine = tf.fused_gemm_bias_gelu(cases[f"{g}/A"], cases[f"{g}/B"], cases[f"{g}/bias"])
    assert np.abs(mine - ref[f"{g}/C"]).max() < 1e-4


@pytest.mark.parametrize("tag", ["a", "b"])
def test_fp16_gemm_matches_the_reference_kernels(tf, reference_outputs, tag):
    cases, ref = reference_outputs
    g = f"gemm_f16_{tag}"
    assert int(ref[f"{g}/status"][0]) == 0
    mine = tf.fused_gemm_bias_gelu(cases[f"{g}/A"], cases[f"{g}/B"], cases[f"{g}/bias"]).astype(np.float64)
    theirs = ref[f"{g}/C"].astype(np.float64)
    assert np.isfinite(theirs).all()
    err = np.abs(mine - theirs)
    assert (err <= 1e-3 + 1e-2 * np.abs(theirs)).all(), float(err.max())
    print(f"FP16 {tag}: max |this - reference| = {err.max():.3e}")


def test_int8_gemm_matches_the_reference_kernels(tf, reference_outputs):
    cases, ref = reference_outputs
    g = "gemm_i8_a"
    assert int(ref[f"{g}/status"][0]) == 0
    sA, sB = (float(v) for v in cases[f"{g}/scales"])
    mine = tf.fused_gemm_bias_gelu(cases[f"{g}/A"], cases[f"{g}/B"], cases[f"{g}/bias"], scales=(sA, sB),
                                   out_dtype=np.float32)
    theirs = ref[f"{g}/C"]
    assert np.isfinite(theirs).all()
    assert np.abs(mine - theirs).max() <= 1e-3 * np.abs(theirs).max()


@pytest.mark.parametrize("tag,tol", [("f32_p0", 1e-4), ("f16_p0", None)])
def test_softmax_matches_the_reference_kernels(tf, reference_outputs, tag, tol):
    cases, ref = reference_outputs
    g = f"softmax_{tag}"
    assert int(ref[f"{g}/status"][0]) == 0
    out, mask = tf.fused_softmax_dropout(cases[f"{g}/x"], dropout_prob=0.0)
    theirs = ref[f"{g}/out"].astype(np.float64)
    err = np.abs(out.astype(np.float64) - theirs)
    if tol is None:      # FP16 storage: two ulps of the reference's value
        assert (err <= 2.0 * np.maximum(np.abs(theirs) * 2.0 ** -10, 2.0 ** -24)).all(), float(err.max())
    else:
        assert err.max() < tol
    assert (mask == 1).all() and (ref[f"{g}/mask"] == 1).all()


def test_dropout_statistics_match_the_reference_kernels(tf, reference_outputs):
    cases, ref = reference_outputs
    g = "softmax_f16_p02"
    assert int(ref[f"{g}/status"][0]) == 0
    x = cases[f"{g}/x"]
    out, mask = tf.fused_softmax_dropout(x, dropout_prob=0.2, seed=5)
    plain, _ = tf.fused_softmax_dropout(x, dropout_prob=0.0)
    for o, m, name in ((out, mask, "this library"), (ref[f"{g}/out"], ref[f"{g}/mask"], "the reference")):
        keep = float(m.mean())
        assert abs(keep - 0.8) < 0.05, (name, keep)       # reference src/tests/test_softmax_dropout.cu:231-246
        kept = m == 1
        want = plain.astype(np.float64) / 0.8
        assert np.abs(o.astype(np.float64)[kept] - want[kept]).max() <= 2e-3, name
        assert (o[~kept] == 0).all(), name


# ------------------------------------------------------------ benchmark sizes
@pytest.fixture(scope="module")
def reference_outputs_full(tmp_path_factory):
    """The benchmark configurations themselves through the reference's kernels:
    configuration 1 and 2 whole, a 1024-row band of configuration 3, a quarter of
    the batch of configuration 4 (same generators, same seeds)."""
    from tensorfuse_b200 import workloads
    c = {}
    x, w, b = workloads.gemm_fp32_quickstart()
    c["gemm_f32_cfg1/A"], c["gemm_f32_cfg1/B"], c["gemm_f32_cfg1/bias"] = x.reshape(-1, x.shape[-1]), w, b
    a, w, b = workloads.gemm_fp16_ffn(seed=1)
    c["gemm_f16_cfg2/A"], c["gemm_f16_cfg2/B"], c["gemm_f16_cfg2/bias"] = a, w, b
    a, w, b, sa, sw = workloads.gemm_int8(seed=2)
    c["gemm_i8_cfg3/A"], c["gemm_i8_cfg3/B"], c["gemm_i8_cfg3/bias"] = a[:1024], w, b.astype(np.float32)
    c["gemm_i8_cfg3/scales"] = np.array([1.0 / sa, 1.0 / sw], dtype=np.float32)    # the reference's q = x * scale
    s = workloads.attention_scores(seed=3, batch=8, masked=True)
    c["softmax_cfg4/x"], c["softmax_cfg4/p"], c["softmax_cfg4/seed"] = s, np.array([0.0], np.float32), np.array([3], np.uint64)
    d = tmp_path_factory.mktemp("reflib_full")
    src, dst = str(d / "in.npz"), str(d / "out.npz")
    np.savez(src, **c)
    r = subprocess.run([sys.executable, RUNNER, "cases", src, dst], capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return c, np.load(dst)


def test_benchmark_configurations_against_the_reference_kernels(tf, reference_outputs_full):
    c, ref = reference_outputs_full
    for g in ("gemm_f32_cfg1", "gemm_f16_cfg2", "gemm_i8_cfg3", "softmax_cfg4"):
        assert int(ref[f"{g}/status"][0]) == 0, g
    # configuration 1, whole output
    mine = tf.fused_gemm_bias_gelu(c["gemm_f32_cfg1/A"], c["gemm_f32_cfg1/B"], c["gemm_f32_cfg1/bias"])
    assert np.abs(mine - ref["gemm_f32_cfg1/C"]).max() < 1e-4
    # configuration 2, whole output
    mine = tf.fused_gemm_bias_gelu(c["gemm_f16_cfg2/A"], c["gemm_f16_cfg2/B"], c["gemm_f16_cfg2/bias"]).astype(np.float32)
    theirs = ref["gemm_f16_cfg2/C"].astype(np.float32)
    err = np.abs(mine - theirs)
    assert (err <= 1e-3 + 1e-2 * np.abs(theirs)).all(), float(err.max())
    # configuration 3, 1024 rows, the reference's scaled FP32 convention
    sA, sB = (float(v) for v in c["gemm_i8_cfg3/scales"])
    mine = tf.fused_gemm_bias_gelu(c["gemm_i8_cfg3/A"], c["gemm_i8_cfg3/B"], c["gemm_i8_cfg3/bias"], scales=(sA, sB),
                                   out_dtype=np.float32)
    theirs = ref["gemm_i8_cfg3/C"]
    assert np.abs(mine - theirs).max() <= 1e-3 * np.abs(theirs).max()
    # configuration 4 (8 of 32 batch items, key padding as -inf), p = 0
    out, mask = tf.fused_softmax_dropout(c["softmax_cfg4/x"], dropout_prob=0.0)
    theirs = ref["softmax_cfg4/out"].astype(np.float32)
    err = np.abs(out.astype(np.float32) - theirs)
    assert (err <= 2.0 * np.maximum(np.abs(theirs) * 2.0 ** -10, 2.0 ** -24)).all(), float(err.max())
    assert ((out == 0) | (mask == 1)).all()

"""This library against golden OUTPUTS of the reference's own GPU kernels.

tests/golden/reference_gpu_kernels.npz was produced on a B200 by
tests/golden/gen_reference_gpu_golden.py, which runs the reference's library
(compiled from a checkout for sm_100a) on small seeded operands.  The operands
are regenerated here from the same seed (and checked against the stored
checksum).  Tolerances as in tests/test_reference_library_gpu.py: FP32 GEMM 1e-4
absolute; FP16 GEMM 1e-2 relative + 1e-3 absolute (the reference rounds the
pre-activation to FP16 first); INT8 in the reference's scaled FP32 convention
1e-3 of the largest magnitude; softmax 1e-4 (FP32) / two FP16 ulps.
"""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import gen_reference_gpu_golden as gen  # noqa: E402

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.exists(gen.GOLDEN), reason="golden vectors of the reference's kernels absent")]


@pytest.fixture(scope="module")
def golden():
    c = gen.cases()
    g = np.load(gen.GOLDEN)
    assert bytes(g["inputs_sha256"]).decode() == gen.checksum(c), "the seeded operands no longer match the golden file"
    for k in g.files:
        if k.endswith("/status"):
            assert int(g[k][0]) == 0, k
    return c, g


def test_fp32_gemm(tf, golden):
    c, g = golden
    mine = tf.fused_gemm_bias_gelu(c["gemm_f32_g/A"], c["gemm_f32_g/B"], c["gemm_f32_g/bias"])
    assert np.abs(mine - g["gemm_f32_g/C"]).max() < 1e-4


def test_fp16_gemm(tf, golden):
    c, g = golden
    mine = tf.fused_gemm_bias_gelu(c["gemm_f16_g/A"], c["gemm_f16_g/B"], c["gemm_f16_g/bias"]).astype(np.float64)
    theirs = g["gemm_f16_g/C"].astype(np.float64)
    assert (np.abs(mine - theirs) <= 1e-3 + 1e-2 * np.abs(theirs)).all()


def test_int8_gemm_scaled_convention(tf, golden):
    c, g = golden
    sA, sB = (float(v) for v in c["gemm_i8_g/scales"])
    mine = tf.fused_gemm_bias_gelu(c["gemm_i8_g/A"], c["gemm_i8_g/B"], c["gemm_i8_g/bias"], scales=(sA, sB),
                                   out_dtype=np.float32)
    theirs = g["gemm_i8_g/C"]
    assert np.abs(mine - theirs).max() <= 1e-3 * np.abs(theirs).max()


@pytest.mark.parametrize("tag", ["f32_g", "f16_g"])
def test_softmax(tf, golden, tag):
    c, g = golden
    out, mask = tf.fused_softmax_dropout(c[f"softmax_{tag}/x"], dropout_prob=0.0)
    theirs = g[f"softmax_{tag}/out"].astype(np.float64)
    err = np.abs(out.astype(np.float64) - theirs)
    if tag == "f32_g":
        assert err.max() < 1e-4
    else:
        assert (err <= 2.0 * np.maximum(np.abs(theirs) * 2.0 ** -10, 2.0 ** -24)).all()
    assert (mask == 1).all()

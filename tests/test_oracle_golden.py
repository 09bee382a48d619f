"""The CPU oracle against the reference's own numbers.

Fixtures in tests/golden/ were produced by importing the reference's numpy
oracle (see tests/golden/gen_golden.py); the known-answer values come from the
reference's C++ tests.  Nothing here needs a GPU.
"""
import math

import numpy as np
import pytest

SIZES = [(1, 1, 1), (8, 16, 32), (16, 32, 64), (32, 64, 128)]


@pytest.mark.parametrize("M,N,K", SIZES)
def test_gemm_bias_gelu_matches_reference_numpy_oracle(oracle, golden, M, N, K):
    tag = f"gemm_{M}x{N}x{K}"
    A, B, bias, C = (golden[tag + s] for s in ("_A", "_B", "_bias", "_C"))
    got = oracle.gemm_bias_gelu_f32(A, B, bias)
    # tolerance of the reference's own test (test_mathematical_verification.py:132)
    np.testing.assert_allclose(got, C, rtol=1e-4, atol=1e-4)
    # and the numpy twin reproduces the fixture to rounding
    np.testing.assert_allclose(oracle.np_gemm_bias_gelu(A, B, bias), C, rtol=1e-6, atol=1e-7)


def test_gelu_known_points(oracle, golden):
    pts, vals = golden["gelu_points"], golden["gelu_values"]
    got = oracle.gelu(pts)
    np.testing.assert_allclose(got, vals, rtol=1e-6, atol=1e-7)
    assert abs(got[4]) < 1e-5          # GELU(0) = 0 to 5 places
    assert got[6] > 0 and got[0] < 0.1  # GELU(1) > 0, GELU(-3) ~ 0
    # C-API smoke value GELU(1*2+0.5) (reference test_c_api_debug.cpp:163-170)
    assert abs(float(oracle.gelu(np.array([2.5], np.float32))[0]) - float(golden["gelu_2p5"][0])) < 1e-6
    assert abs(float(golden["gelu_2p5"][0]) - 2.4851) < 1e-3


def test_all_point_one_case_is_finite_and_small(oracle):
    # reference test_working_kernel.cu:86-135: 8x16x32 of 0.1 -> finite, |x| < 10
    A = np.full((8, 32), 0.1, np.float32); B = np.full((32, 16), 0.1, np.float32)
    out = oracle.gemm_bias_gelu_f32(A, B, np.full(16, 0.1, np.float32))
    assert np.all(np.isfinite(out)) and np.all(np.abs(out) < 10)
    want = 0.42 * 0.5 * (1 + math.tanh(0.7978845608028654 * (0.42 + 0.044715 * 0.42 ** 3)))
    np.testing.assert_allclose(out, want, rtol=1e-5)


def test_alpha_beta_grid(oracle):
    # (alpha, beta) pairs of reference test_gemm_edge_cases.cu:171-181
    r = np.random.default_rng(42)
    A = r.uniform(-0.5, 0.5, (16, 24)).astype(np.float32)
    B = r.uniform(-0.5, 0.5, (24, 20)).astype(np.float32)
    b = r.uniform(-0.5, 0.5, 20).astype(np.float32)
    for alpha, beta in [(1, 1), (0, 1), (1, 0), (0, 0), (2, 0.5), (-1, 1), (1, -1), (0.5, 2), (-0.5, -0.5)]:
        got = oracle.gemm_bias_gelu_f32(A, B, b, alpha, beta)
        np.testing.assert_allclose(got, oracle.np_gemm_bias_gelu(A.astype(np.float64), B.astype(np.float64), b, alpha, beta),
                                   rtol=1e-4, atol=1e-5)


def test_softmax_matches_reference_numpy_oracle(oracle, golden):
    x, y = golden["softmax_in"], golden["softmax_out"]
    np.testing.assert_allclose(oracle.softmax_ref_f32(x), y, rtol=1e-5, atol=1e-7)
    exact, mask = oracle.softmax_dropout_exact(x, p=0.0)
    assert mask.min() == 1
    # reference tolerance (test_mathematical_verification.py:223) and much tighter in practice
    np.testing.assert_allclose(exact, y, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(exact, y, rtol=2e-6, atol=1e-9)
    np.testing.assert_allclose(exact.sum(-1), 1.0, rtol=1e-5)


@pytest.mark.parametrize("vec,warps", [(8, 1), (8, 8), (1, 1), (1, 8)])
def test_exact_softmax_schedules_agree_to_rounding(oracle, vec, warps):
    r = np.random.default_rng(7)
    x = (r.standard_normal((3, 1000)) * 2).astype(np.float32)
    base = oracle.np_softmax(x.astype(np.float64))
    got, _ = oracle.softmax_dropout_exact(x, vec=vec, warps=warps)
    np.testing.assert_allclose(got, base, rtol=3e-6, atol=1e-10)


def test_exact_softmax_masked_and_empty_rows(oracle):
    x = np.zeros((3, 16), np.float16)
    x[0, 8:] = -np.inf            # half masked
    x[1, :] = -np.inf             # fully masked -> zeros by definition
    x[2, :] = np.linspace(-4, 4, 16)
    y, m = oracle.softmax_dropout_exact(x)
    assert np.all(y[0, 8:] == 0) and np.allclose(y[0, :8].astype(np.float32), 0.125, rtol=1e-3)
    assert np.all(y[1] == 0) and not np.any(np.isnan(y))
    assert m.min() == 1


def test_philox_known_answers(oracle):
    # Known-answer vectors of the Random123 distribution for philox4x32-10.
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
            (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for ctr, key, want in kat:
        assert tuple(int(v) for v in oracle.philox4x32_10(ctr, key)) == want


def test_dropout_mask_statistics_and_sharding(oracle):
    n, p, seed = 1 << 20, 0.1, 12345
    m = oracle.dropout_mask(n, p, seed)
    assert abs(m.mean() - 0.9) < 4 * math.sqrt(0.09 / n) + 1e-4
    # a shard draws exactly what it would draw as part of the whole
    part = oracle.dropout_mask(4096, p, seed, first_idx=8 * 1000)
    assert np.array_equal(part, m[8000:8000 + 4096])
    assert oracle.dropout_threshold(0.0) == 0 and oracle.dropout_threshold(1.0) == 32768
    assert oracle.dropout_mask(64, 1.0, 1).max() == 0 and oracle.dropout_mask(64, 0.0, 1).min() == 1
    # dropout semantics: kept values are softmax / (1 - p), dropped are 0
    x = np.random.default_rng(3).standard_normal((4, 64)).astype(np.float32)
    y0, _ = oracle.softmax_dropout_exact(x, p=0.0)
    y, mk = oracle.softmax_dropout_exact(x, p=0.25, seed=9)
    assert np.all(y[mk == 0] == 0)
    np.testing.assert_allclose(y[mk == 1], y0[mk == 1] / 0.75, rtol=3e-7)


def test_int8_paths(oracle, golden):
    A, B, bias = golden["int8_A"], golden["int8_B"], golden["int8_bias"]
    sA, sB = (float(v) for v in golden["int8_scales"])
    acc = oracle.gemm_i8_acc(A, B)
    assert np.array_equal(acc, A.astype(np.int64) @ B.astype(np.int64))
    out = oracle.i8_epilogue_legacy_f32(acc, bias, sA, sB)
    ref = golden["int8_fp32_reference"]
    # the reference's own criterion (test_int8_tensor_cores.py:92-105)
    rel = np.max(np.abs(ref - out / (sA * sB))) / np.max(np.abs(ref))
    assert rel < 0.15
    # multiply convention
    qa = 1.0 / sA; qb = 1.0 / sB
    h = oracle.i8_epilogue_f16(acc, bias.astype(np.float16), qa, qb)
    want = oracle.np_gelu(acc.astype(np.float64) * np.float32(qa * qb) + bias.astype(np.float16).astype(np.float64))
    assert oracle.f16_parity_violations(h, want.astype(np.float16)) == 0


def test_fp16_gemm_single_rounding(oracle):
    r = np.random.default_rng(1)
    A = r.standard_normal((24, 40)).astype(np.float16)
    B = (r.standard_normal((40, 32)) / 6).astype(np.float16)
    b = (r.standard_normal(32) * 0.02).astype(np.float16)
    got = oracle.gemm_bias_gelu_f16(A, B, b)
    want = oracle.np_gemm_bias_gelu(A.astype(np.float64), B.astype(np.float64), b.astype(np.float64))
    assert oracle.f16_ulp_distance(got, want.astype(np.float16)).max() <= 1


# ------------------------------------------------- the reference's GPU kernels
def _reference_gpu_golden():
    import os
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(here, "golden"))
    import gen_reference_gpu_golden as gen
    if not os.path.exists(gen.GOLDEN):
        pytest.skip("golden vectors of the reference's kernels absent")
    c, g = gen.cases(), np.load(gen.GOLDEN)
    assert bytes(g["inputs_sha256"]).decode() == gen.checksum(c)
    return c, g


def test_oracle_matches_outputs_of_the_reference_gpu_kernels(oracle):
    """tests/golden/reference_gpu_kernels.npz holds what the reference's own library
    (compiled from a checkout for sm_100a) wrote on a B200 for seeded operands
    (tests/golden/gen_reference_gpu_golden.py).  The CPU oracle must agree with it:
    FP32 GEMM at the reference's 1e-4; FP16 GEMM within 1e-2 relative + 1e-3 absolute
    (the reference rounds the pre-activation to FP16, the oracle rounds once); INT8 in the
    reference's scaled FP32 convention within 1e-3 of the largest magnitude (the reference
    is built with --use_fast_math); softmax within 1e-4 / two FP16 ulps."""
    c, g = _reference_gpu_golden()
    got = oracle.gemm_bias_gelu_f32(c["gemm_f32_g/A"], c["gemm_f32_g/B"], c["gemm_f32_g/bias"])
    assert np.abs(got - g["gemm_f32_g/C"]).max() < 1e-4
    got = oracle.gemm_bias_gelu_f16(c["gemm_f16_g/A"], c["gemm_f16_g/B"], c["gemm_f16_g/bias"]).astype(np.float64)
    theirs = g["gemm_f16_g/C"].astype(np.float64)
    assert (np.abs(got - theirs) <= 1e-3 + 1e-2 * np.abs(theirs)).all()
    sA, sB = (float(v) for v in c["gemm_i8_g/scales"])
    acc = oracle.gemm_i8_acc(c["gemm_i8_g/A"], c["gemm_i8_g/B"])
    got = oracle.i8_epilogue_legacy_f32(acc, c["gemm_i8_g/bias"], sA, sB)
    theirs = g["gemm_i8_g/C"]
    assert np.abs(got - theirs).max() <= 1e-3 * np.abs(theirs).max()
    got = oracle.softmax_ref_f32(c["softmax_f32_g/x"])
    assert np.abs(got - g["softmax_f32_g/out"]).max() < 1e-4
    got = oracle.softmax_ref_f16(c["softmax_f16_g/x"])[0].astype(np.float64)
    theirs = g["softmax_f16_g/out"].astype(np.float64)
    assert (np.abs(got - theirs) <= 2.0 * np.maximum(np.abs(theirs) * 2.0 ** -10, 2.0 ** -24)).all()

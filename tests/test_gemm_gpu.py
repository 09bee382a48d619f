"""fused_gemm_bias_gelu on the GPU against the CPU oracle, through the C ABI.

Tolerances
  FP32 : 1e-4 absolute (1e-2 for the extreme-value fills), the reference's own
         (src/tests/test_kernels.cu:139, test_gemm_edge_cases.cu:383)
  FP16 : 1e-2 relative / 1e-3 absolute against the FP32-accumulate oracle
  INT8 : INT32 accumulator bit-exact; FP16 result within 1 FP16 ulp of the oracle
         (absolute 2^-22 below the smallest normal FP16, where the oracle's FP32
         tanh form itself cancels); reference-convention FP32 result 1e-5 relative
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FP16_RTOL, FP16_ATOL = 1e-2, 1e-3


def _close_f16(got, want):
    g = got.astype(np.float32); w = want.astype(np.float32)
    bad = np.abs(g - w) > (FP16_ATOL + FP16_RTOL * np.abs(w))
    return int(bad.sum())


# ------------------------------------------------------------------- FP32
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (8, 16, 32), (16, 32, 64), (32, 64, 128), (64, 128, 256),
                                   (1, 16, 1), (16, 1, 16), (129, 130, 67), (256, 1024, 2048)])
def test_fp32_sizes(tf, oracle, M, N, K):
    from gpu_util import gemm_wrapper
    r = np.random.default_rng(42)
    A = r.uniform(-0.5, 0.5, (M, K)).astype(np.float32)
    B = r.uniform(-0.5, 0.5, (K, N)).astype(np.float32)
    b = r.uniform(-0.5, 0.5, N).astype(np.float32)
    st, out = gemm_wrapper("fused_gemm_bias_gelu_fp32_wrapper", A, B, b, torch.float32)
    assert st == 0
    np.testing.assert_allclose(out, oracle.gemm_bias_gelu_f32(A, B, b), rtol=1e-4, atol=1e-4)


def test_fp32_reference_fixtures(tf, golden):
    from gpu_util import gemm_wrapper
    for (M, N, K) in [(1, 1, 1), (8, 16, 32), (16, 32, 64), (32, 64, 128)]:
        tag = f"gemm_{M}x{N}x{K}"
        st, out = gemm_wrapper("optimized_fused_gemm_bias_gelu_fp32_wrapper", golden[tag + "_A"],
                               golden[tag + "_B"], golden[tag + "_bias"], torch.float32)
        assert st == 0
        np.testing.assert_allclose(out, golden[tag + "_C"], rtol=1e-4, atol=1e-4)
    # GELU known points through A = [[1]] (reference test_mathematical_verification.py:225-260)
    pts = golden["gelu_points"]
    st, out = gemm_wrapper("fused_gemm_bias_gelu_fp32_wrapper", np.ones((1, 1), np.float32), pts.reshape(1, -1),
                           np.zeros(pts.size, np.float32), torch.float32)
    np.testing.assert_allclose(out.ravel(), golden["gelu_values"], rtol=1e-4, atol=1e-4)
    assert abs(out.ravel()[4]) < 1e-5
    # GELU(1*2 + 0.5) (reference test_c_api_debug.cpp:163-170)
    st, out = gemm_wrapper("fused_gemm_bias_gelu_fp32_wrapper", np.array([[1.0]], np.float32),
                           np.array([[2.0]], np.float32), np.array([0.5], np.float32), torch.float32)
    assert abs(float(out[0, 0]) - float(golden["gelu_2p5"][0])) < 1e-4


@pytest.mark.parametrize("alpha,beta", [(1, 1), (0, 1), (1, 0), (0, 0), (2, 0.5), (-1, 1), (1, -1), (0.5, 2),
                                        (-0.5, -0.5)])
def test_fp32_alpha_beta(tf, oracle, alpha, beta):
    from gpu_util import gemm_wrapper
    r = np.random.default_rng(42)
    A = r.uniform(-0.5, 0.5, (48, 40)).astype(np.float32)
    B = r.uniform(-0.5, 0.5, (40, 56)).astype(np.float32)
    b = r.uniform(-0.5, 0.5, 56).astype(np.float32)
    st, out = gemm_wrapper("fused_gemm_bias_gelu_fp32_wrapper", A, B, b, torch.float32, alpha, beta)
    assert st == 0
    np.testing.assert_allclose(out, oracle.gemm_bias_gelu_f32(A, B, b, alpha, beta), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("fill", ["zeros", "ones", "p100", "m100", "tiny", "alt1000"])
def test_fp32_extreme_values(tf, oracle, fill):
    from gpu_util import gemm_wrapper
    M, N, K = 32, 48, 40
    val = {"zeros": 0.0, "ones": 1.0, "p100": 100.0, "m100": -100.0, "tiny": 1e-6}.get(fill)
    if val is None:
        A = np.where(np.arange(M * K) % 2 == 0, 1000.0, -1000.0).astype(np.float32).reshape(M, K)
        B = np.where(np.arange(K * N) % 2 == 0, 1000.0, -1000.0).astype(np.float32).reshape(K, N)
    else:
        A = np.full((M, K), val, np.float32); B = np.full((K, N), val, np.float32)
    b = np.zeros(N, np.float32)
    st, out = gemm_wrapper("fused_gemm_bias_gelu_fp32_wrapper", A, B, b, torch.float32)
    assert st == 0 and np.all(np.isfinite(out))
    np.testing.assert_allclose(out, oracle.gemm_bias_gelu_f32(A, B, b), rtol=1e-5, atol=1e-2)


# ------------------------------------------------------------------- FP16
FP16_SHAPES = [(128, 256, 64), (256, 512, 128), (128, 256, 1024), (384, 768, 192),
               (100, 264, 72), (1, 8, 8), (130, 8, 24), (520, 1032, 200),     # tails in M, N and K
               (2048, 4096, 1024)]


@pytest.mark.parametrize("M,N,K", FP16_SHAPES)
def test_fp16_tensor_core_path(tf, oracle, M, N, K):
    from gpu_util import gemm_wrapper
    r = np.random.default_rng(M + N + K)
    A = r.standard_normal((M, K)).astype(np.float16)
    B = (r.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16)
    b = (r.standard_normal(N) * 0.02).astype(np.float16)
    st, out = gemm_wrapper("fused_gemm_bias_gelu_fp16_wrapper", A, B, b, torch.float16)
    assert st == 0
    want = oracle.gemm_bias_gelu_f16(A, B, b)
    assert _close_f16(out, want) == 0
    # in practice the two agree to the last place almost everywhere
    assert oracle.f16_parity_violations(out, want, max_ulp=2, tiny_abs=2.0 ** -20) <= out.size // 1000


@pytest.mark.parametrize("M,N,K", [(33, 17, 9), (64, 100, 36), (7, 12, 8)])
def test_fp16_unaligned_shapes_use_cuda_cores(tf, oracle, M, N, K):
    from gpu_util import gemm_wrapper
    r = np.random.default_rng(9)
    A = r.standard_normal((M, K)).astype(np.float16)
    B = (r.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16)
    b = (r.standard_normal(N) * 0.02).astype(np.float16)
    st, out = gemm_wrapper("optimized_fused_gemm_bias_gelu_fp16_wrapper", A, B, b, torch.float16)
    assert st == 0 and _close_f16(out, oracle.gemm_bias_gelu_f16(A, B, b)) == 0


def test_fp16_alpha_beta_and_determinism(tf, oracle):
    from gpu_util import gemm_wrapper
    r = np.random.default_rng(3)
    A = r.standard_normal((256, 128)).astype(np.float16)
    B = (r.standard_normal((128, 256)) / 11).astype(np.float16)
    b = (r.standard_normal(256) * 0.5).astype(np.float16)
    for alpha, beta in [(1, 1), (0.5, 2), (-1, 1), (1, 0)]:
        st, out = gemm_wrapper("fused_gemm_bias_gelu_fp16_wrapper", A, B, b, torch.float16, alpha, beta)
        assert st == 0 and _close_f16(out, oracle.gemm_bias_gelu_f16(A, B, b, alpha, beta)) == 0
    a1 = gemm_wrapper("fused_gemm_bias_gelu_fp16_wrapper", A, B, b, torch.float16)[1]
    a2 = gemm_wrapper("fused_gemm_bias_gelu_fp16_wrapper", A, B, b, torch.float16)[1]
    assert np.array_equal(a1.view(np.uint16), a2.view(np.uint16))


def test_fp16_full_ffn_shape(tf, oracle):
    """Config 2 at full size; the oracle is evaluated on a sample of rows."""
    from gpu_util import L, check_watchdog, dev, host, stream
    from tensorfuse_b200 import workloads
    A, B, b = workloads.gemm_fp16_ffn()
    M, K = A.shape; N = B.shape[1]
    dA, dB, db = dev(A), dev(B), dev(b)
    dC = torch.empty((M, N), dtype=torch.float16, device="cuda")
    assert L.fused_gemm_bias_gelu_fp16_wrapper(dA.data_ptr(), dB.data_ptr(), db.data_ptr(), dC.data_ptr(), M, N, K,
                                               1.0, 1.0, stream()) == 0
    check_watchdog()
    rows = np.sort(np.random.default_rng(0).choice(M, 96, replace=False))
    want = oracle.gemm_bias_gelu_f16(A[rows], B, b)
    got = host(dC[torch.from_numpy(rows).cuda()])
    assert _close_f16(got, want) == 0
    # row-sharding (what the multi-GPU path does) reproduces the whole bit for bit
    dC2 = torch.empty_like(dC)
    for r0, cnt in zip(*tf.plan_shards(M, 3, 128)):
        assert L.fused_gemm_bias_gelu_fp16_wrapper(dA.data_ptr() + 2 * r0 * K, dB.data_ptr(), db.data_ptr(),
                                                   dC2.data_ptr() + 2 * r0 * N, cnt, N, K, 1.0, 1.0, stream()) == 0
    check_watchdog()
    assert torch.equal(dC, dC2)


# ------------------------------------------------------------------- INT8
INT8_SHAPES = [(128, 256, 128), (256, 512, 256), (128, 256, 4096), (100, 272, 144), (1, 16, 16),
               (300, 1040, 400), (1024, 2048, 1024)]


def _int8_case(M, N, K, seed):
    r = np.random.default_rng(seed)
    A = r.integers(-127, 128, (M, K), dtype=np.int8)
    B = r.integers(-127, 128, (K, N), dtype=np.int8)
    return A, B


@pytest.mark.parametrize("M,N,K", INT8_SHAPES)
def test_int8_accumulator_bit_exact(tf, oracle, M, N, K):
    from gpu_util import DT, gemm_int8
    A, B = _int8_case(M, N, K, M * 7 + K)
    st, acc = gemm_int8(A, B, np.zeros(N, np.float32), (1.0, 1.0), DT.FLOAT32, torch.int32, tf.INT8_RAW)
    assert st == 0
    assert np.array_equal(acc, oracle.gemm_i8_acc(A, B))


def test_int8_extreme_operands(tf, oracle):
    from gpu_util import DT, gemm_int8
    M, N, K = 128, 256, 1024
    for a_val, b_val in [(127, 127), (-127, 127), (-128, -128), (-128, 127)]:
        A = np.full((M, K), a_val, np.int8); B = np.full((K, N), b_val, np.int8)
        st, acc = gemm_int8(A, B, np.zeros(N, np.float32), (1.0, 1.0), DT.FLOAT32, torch.int32, tf.INT8_RAW)
        assert st == 0 and np.all(acc == a_val * b_val * K)


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (100, 272, 144), (1024, 2048, 1024)])
def test_int8_dequant_fp16_within_one_ulp(tf, oracle, M, N, K):
    from gpu_util import DT, gemm_int8
    from tensorfuse_b200 import workloads
    r = np.random.default_rng(2)
    A, sa = workloads.quantize_sym_int8(r.standard_normal((M, K)).astype(np.float32))
    B, sb = workloads.quantize_sym_int8((r.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32))
    bias = (r.standard_normal(N) * 0.02).astype(np.float16)
    st, out = gemm_int8(A, B, bias, (sa, sb), DT.FLOAT16, torch.float16, tf.INT8_DEQUANT)
    assert st == 0
    acc = oracle.gemm_i8_acc(A, B)
    want = oracle.i8_epilogue_f16(acc, bias, sa, sb)
    assert oracle.f16_parity_violations(out, want, max_ulp=1) == 0
    # and against the formula evaluated in float64 ("truth"), same bound
    truth = oracle.np_gelu(acc.astype(np.float64) * float(np.float32(sa) * np.float32(sb)) +
                           bias.astype(np.float64)).astype(np.float16)
    assert oracle.f16_parity_violations(out, truth, max_ulp=1) == 0


def test_int8_reference_convention(tf, oracle, golden):
    from gpu_util import gemm_wrapper
    A, B, bias = golden["int8_A"], golden["int8_B"], golden["int8_bias"]
    sA, sB = (float(v) for v in golden["int8_scales"])
    st, out = gemm_wrapper("fused_gemm_bias_gelu_int8_wrapper_with_scales", A, B, bias, torch.float32, 1.0, 1.0,
                           (sA, sB))
    assert st == 0
    want = oracle.i8_epilogue_legacy_f32(oracle.gemm_i8_acc(A, B), bias, sA, sB)
    # absolute part: FP32 cancellation noise of 1 + tanh (~1e-7) times the output scale sA*sB
    np.testing.assert_allclose(out, want, rtol=1e-5, atol=4e-7 * sA * sB)
    ref = golden["int8_fp32_reference"]     # the reference test's own criterion: 15 % of max
    assert np.max(np.abs(ref - out / (sA * sB))) / np.max(np.abs(ref)) < 0.15
    st, out1 = gemm_wrapper("fused_gemm_bias_gelu_int8_wrapper", A, B, bias, torch.float32)
    np.testing.assert_allclose(out1, oracle.i8_epilogue_legacy_f32(oracle.gemm_i8_acc(A, B), bias, 1.0, 1.0),
                               rtol=1e-5, atol=1e-3)


def test_int8_unaligned_shape(tf, oracle):
    from gpu_util import DT, gemm_int8
    A, B = _int8_case(37, 21, 19, 5)
    st, acc = gemm_int8(A, B, np.zeros(21, np.float32), (1.0, 1.0), DT.FLOAT32, torch.int32, tf.INT8_RAW)
    assert st == 0 and np.array_equal(acc, oracle.gemm_i8_acc(A, B))


def test_int8_full_size_sampled(tf, oracle):
    """Config 3 at full size (M 8192, K 4096, N 16384): accumulators and FP16
    results of a sample of rows against the oracle."""
    from gpu_util import DT, L, check_watchdog, dev, host, stream
    from tensorfuse_b200 import workloads
    A, B, bias, sa, sb = workloads.gemm_int8()
    M, K = A.shape; N = B.shape[1]
    dA, dB, db = dev(A), dev(B), dev(bias)
    dC = torch.empty((M, N), dtype=torch.float16, device="cuda")
    assert L.tensorfuse_b200_gemm_int8(dA.data_ptr(), dB.data_ptr(), db.data_ptr(), dC.data_ptr(), M, N, K, sa, sb,
                                       int(DT.FLOAT16), int(DT.FLOAT16), tf.INT8_DEQUANT, stream()) == 0
    check_watchdog()
    rows = np.sort(np.random.default_rng(1).choice(M, 48, replace=False))
    acc = oracle.gemm_i8_acc(A[rows], B)
    want = oracle.i8_epilogue_f16(acc, bias, sa, sb)
    got = host(dC[torch.from_numpy(rows).cuda()])
    assert oracle.f16_parity_violations(got, want, max_ulp=1) == 0
    dI = torch.empty((M, N), dtype=torch.int32, device="cuda")
    assert L.tensorfuse_b200_gemm_int8(dA.data_ptr(), dB.data_ptr(), db.data_ptr(), dI.data_ptr(), M, N, K, 1.0, 1.0,
                                       int(DT.FLOAT32), int(DT.INT32), tf.INT8_RAW, stream()) == 0
    check_watchdog()
    assert np.array_equal(host(dI[torch.from_numpy(rows).cuda()]), acc)


# ------------------------------------------------------- linear epilogue
@pytest.mark.parametrize("dtype,M,N,K", [(np.float16, 384, 512, 256), (np.float16, 100, 264, 72),
                                         (np.float16, 33, 17, 9), (np.float32, 65, 70, 33)])
def test_bias_only_epilogue(tf, dtype, M, N, K):
    """activation NONE (the FFN-down form): alpha*A*B + beta*bias without GELU."""
    from gpu_util import DT, L, check_watchdog, dev, host, stream
    r = np.random.default_rng(M)
    A = r.standard_normal((M, K)).astype(dtype)
    B = (r.standard_normal((K, N)) / np.sqrt(K)).astype(dtype)
    b = (r.standard_normal(N) * 0.1).astype(dtype)
    dA, dB, db = dev(A), dev(B), dev(b)
    tdt = torch.float16 if dtype == np.float16 else torch.float32
    for act, alpha, beta in ((0, 1.0, 1.0), (0, 0.125, 0.0), (2, 1.0, 1.0)):
        dC = torch.zeros((M, N), dtype=tdt, device="cuda")
        st = L.tensorfuse_b200_gemm_bias_act(dA.data_ptr(), dB.data_ptr(), db.data_ptr(), dC.data_ptr(), M, N, K,
                                             int(DT.FLOAT16 if dtype == np.float16 else DT.FLOAT32), act, alpha, beta,
                                             stream())
        check_watchdog()
        assert st == 0
        lin = alpha * (A.astype(np.float64) @ B.astype(np.float64)) + beta * b.astype(np.float64)
        want = lin if act == 0 else lin * 0.5 * (1 + np.tanh(0.7978845608028654 * (lin + 0.044715 * lin ** 3)))
        got = host(dC).astype(np.float64)
        tol_r, tol_a = (1e-2, 1e-3) if dtype == np.float16 else (1e-4, 1e-4)
        assert np.all(np.abs(got - want) <= tol_a + tol_r * np.abs(want))
    assert L.tensorfuse_b200_gemm_bias_act(dA.data_ptr(), dB.data_ptr(), db.data_ptr(), dC.data_ptr(), M, N, K,
                                           int(DT.FLOAT16 if dtype == np.float16 else DT.FLOAT32), 1, 1.0, 1.0, None) == 10

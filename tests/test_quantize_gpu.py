"""Device-side INT8 quantisation (tensorfuse_b200_quantize_int8): bit-exact
against the oracle's recipe, and chained into the INT8 GEMM through the
device-resident scales without a host round trip."""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import DT, L, check_watchdog, dev, host, stream

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,dtype", [((1000, 37), np.float32), ((4096, 1024), np.float32), ((513, 129), np.float16),
                                         ((8,), np.float32), ((3,), np.float16), ((2048, 2048), np.float16)])
def test_quantize_matches_oracle(tf, oracle, shape, dtype):
    rng = np.random.default_rng(11)
    x = (rng.standard_normal(shape) * 3).astype(dtype)
    x.flat[0] = 0.5 * np.abs(x).max()              # exact .5 ties appear after the division for some inputs
    q, s = tf.quantize_int8(dev(x))
    wq, ws = oracle.quantize_sym_int8(x)
    assert np.float32(host(s)[0]) == ws
    assert np.array_equal(host(q), wq)
    assert abs(int(host(q).max())) == 127 or abs(int(host(q).min())) == 127


def test_quantize_edge_cases(tf, oracle):
    z = torch.zeros((5, 7), device="cuda")
    q, s = tf.quantize_int8(z)
    assert float(s) == 1.0 and int(q.abs().max()) == 0
    # unaligned base pointer -> scalar path, same result
    x = np.random.default_rng(1).standard_normal(4099).astype(np.float32)
    d = dev(np.concatenate([[0.0], x]).astype(np.float32))[1:]
    q, s = tf.quantize_int8(d)
    wq, ws = oracle.quantize_sym_int8(x)
    assert np.array_equal(host(q), wq) and np.float32(host(s)[0]) == ws
    assert L.tensorfuse_b200_quantize_int8(None, 0, 4, None, None, None) == 1
    assert L.tensorfuse_b200_quantize_int8(d.data_ptr(), int(DT.INT8), 4, q.data_ptr(), s.data_ptr(), None) == 10


def test_quantize_then_int8_gemm_stays_on_device(tf, oracle):
    """activations and weights quantised on the device, scales consumed by the
    GEMM through TensorFuseTensor.scale; raw accumulators bit-exact, FP16 result
    within 1 ulp of the oracle."""
    import tensorfuse_b200 as t
    rng = np.random.default_rng(2)
    M, K, N = 256, 512, 384
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    b = (rng.standard_normal(N) * 0.02).astype(np.float16)
    qa, sa = tf.quantize_int8(dev(A)); qw, sw = tf.quantize_int8(dev(W))
    out = tf.fused_gemm_bias_gelu(qa, qw, dev(b), scales=(sa, sw), out_dtype=torch.float16, int8_mode=t.INT8_DEQUANT)
    check_watchdog()
    oa, osa = oracle.quantize_sym_int8(A); ow, osw = oracle.quantize_sym_int8(W)
    acc = oracle.gemm_i8_acc(oa, ow)
    want = oracle.i8_epilogue_f16(acc, b, float(osa), float(osw))
    assert oracle.f16_parity_violations(host(out), want, max_ulp=1) == 0


@pytest.mark.parametrize("K,N,dtype", [(512, 384, np.float32), (1000, 72, np.float16), (64, 4096, np.float32)])
def test_quantize_columns_matches_oracle(tf, oracle, K, N, dtype):
    rng = np.random.default_rng(12)
    w = (rng.standard_normal((K, N)) * rng.uniform(0.01, 3.0, N)[None, :]).astype(dtype)
    w[:, 5] = 0                                     # an all-zero channel
    q, s = tf.quantize_int8(dev(w), per_column=True)
    wq, ws = oracle.quantize_sym_int8_columns(w)
    assert np.array_equal(host(s), ws)
    assert np.array_equal(host(q), wq)


@pytest.mark.parametrize("M,K,N", [(512, 512, 384), (100, 96, 80), (37, 50, 21)])
def test_channelwise_int8_gemm(tf, oracle, M, K, N):
    """Per-tensor activation scale x per-column weight scales, everything on the
    device; FP16 result within 1 ulp of the float64 formula on the exact accumulators."""
    import tensorfuse_b200 as t
    rng = np.random.default_rng(3)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * rng.uniform(0.02, 1.0, N)[None, :] / np.sqrt(K)).astype(np.float32)
    b = (rng.standard_normal(N) * 0.02).astype(np.float16)
    qa, sa = tf.quantize_int8(dev(A)); qw, sw = tf.quantize_int8(dev(W), per_column=True)
    out = tf.fused_gemm_bias_gelu(qa, qw, dev(b), scales=(sa, sw), out_dtype=torch.float16, int8_mode=t.INT8_DEQUANT)
    check_watchdog()
    oa, osa = oracle.quantize_sym_int8(A); ow, osw = oracle.quantize_sym_int8_columns(W)
    acc = oracle.gemm_i8_acc(oa, ow).astype(np.float64)
    x = acc * (np.float64(osa) * osw.astype(np.float64))[None, :] + b.astype(np.float64)
    ref = (0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))).astype(np.float16)
    assert oracle.f16_parity_violations(host(out), ref, max_ulp=1) == 0

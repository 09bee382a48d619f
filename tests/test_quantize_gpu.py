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

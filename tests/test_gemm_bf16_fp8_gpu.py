"""BF16 and FP8-E4M3 operand variants of the fused GEMM (types the reference
enumerates, src/tensorfuse/types.h:52,56, without kernels).  Oracle: the
reference's gemm_bias_gelu_ref semantics in float64 on the exactly-widened
operands.  Tolerances: BF16 output is one BF16 rounding (2^-8 relative) of an
FP32-accumulated value: |err| <= 1e-2 |want| + 1e-3; FP8 products are exact in
FP32, output FP16: 2e-3 relative + 1e-3."""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import DT, L, check_watchdog, dev, host, stream

pytestmark = pytest.mark.gpu


def bf16_dev(x32):
    return torch.from_numpy(np.ascontiguousarray(x32, np.float32)).cuda().to(torch.bfloat16)


@pytest.mark.parametrize("M,K,N", [(256, 512, 384), (1000, 264, 136), (16384, 1024, 4096), (33, 70, 19)])
@pytest.mark.parametrize("act", [2, 0])
def test_bf16_gemm(tf, oracle, M, K, N, act):
    rng = np.random.default_rng(5)
    A = oracle.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    B = oracle.bf16_round((rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32))
    b = oracle.bf16_round((rng.standard_normal(N) * 0.1).astype(np.float32))
    dA, dB, db = bf16_dev(A), bf16_dev(B), bf16_dev(b)
    dC = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    st = L.tensorfuse_b200_gemm_bias_act(dA.data_ptr(), dB.data_ptr(), db.data_ptr(), dC.data_ptr(), M, N, K,
                                         int(DT.BFLOAT16), act, 1.0, 1.0, stream())
    assert st == 0
    check_watchdog()
    rows = np.unique(np.concatenate([np.arange(min(M, 160)), np.random.default_rng(0).integers(0, M, 64)]))
    want = oracle.gemm_bias_gelu_f64(A[rows], B, b, activation="gelu" if act == 2 else "none")
    got = dC.float().cpu().numpy()[rows]
    assert (np.abs(got - want) <= 1e-2 * np.abs(want) + 1e-3).all()


def test_bf16_struct_entry(tf, oracle):
    import tensorfuse_b200 as t
    rng = np.random.default_rng(6)
    M, K, N = 128, 256, 512
    A = oracle.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    B = oracle.bf16_round((rng.standard_normal((K, N)) / 16).astype(np.float32))
    b = oracle.bf16_round((rng.standard_normal(N) * 0.1).astype(np.float32))
    dA, dB, db = bf16_dev(A), bf16_dev(B), bf16_dev(b)
    dC = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    ct = lambda x: t._c_tensor(x.data_ptr(), tuple(x.shape), DT.BFLOAT16)
    ta, tb, tbias, tc = ct(dA), ct(dB), ct(db), ct(dC)
    assert L.tensorfuse_fused_gemm_bias_gelu(C.byref(ta), C.byref(tb), C.byref(tbias), C.byref(tc), stream()) == 0
    check_watchdog()
    want = oracle.gemm_bias_gelu_f64(A, B, b)
    assert (np.abs(dC.float().cpu().numpy() - want) <= 1e-2 * np.abs(want) + 1e-3).all()


@pytest.mark.parametrize("M,K,N,out", [(256, 512, 384, torch.float16), (8192, 4096, 1024, torch.float16),
                                       (100, 96, 48, torch.float32), (37, 50, 21, torch.float16)])
def test_fp8_gemm(tf, oracle, M, K, N, out):
    rng = np.random.default_rng(7)
    table = oracle.fp8_e4m3_table()
    # byte patterns with |value| <= 8 (exponent field <= 10), no NaN patterns
    def rand_fp8(shape):
        e = rng.integers(0, 11, shape, dtype=np.uint8); m = rng.integers(0, 8, shape, dtype=np.uint8)
        s = rng.integers(0, 2, shape, dtype=np.uint8)
        return (s << 7 | e << 3 | m).astype(np.uint8)
    A8, B8 = rand_fp8((M, K)), rand_fp8((K, N))
    sa, sb = 0.05, 0.02
    b = (rng.standard_normal(N) * 0.1).astype(np.float16 if out == torch.float16 else np.float32)
    dA, dB, db = dev(A8), dev(B8), dev(b)
    dC = torch.zeros((M, N), dtype=out, device="cuda")
    st = L.tensorfuse_b200_gemm_fp8(dA.data_ptr(), dB.data_ptr(), db.data_ptr(), dC.data_ptr(), M, N, K, sa, sb,
                                    int(DT.FLOAT16 if out == torch.float16 else DT.FLOAT32),
                                    int(DT.FLOAT16 if out == torch.float16 else DT.FLOAT32), stream())
    assert st == 0
    check_watchdog()
    rows = np.unique(np.concatenate([np.arange(min(M, 130)), np.random.default_rng(0).integers(0, M, 32)]))
    want = oracle.gemm_bias_gelu_f64(table[A8[rows]], table[B8], b, scale=np.float32(sa) * np.float32(sb))
    got = dC.float().cpu().numpy()[rows]
    assert (np.abs(got - want) <= 2e-3 * np.abs(want) + 1e-3).all()


def test_fp8_struct_entry_with_device_scales(tf, oracle):
    import tensorfuse_b200 as t
    rng = np.random.default_rng(8)
    table = oracle.fp8_e4m3_table()
    M, K, N = 128, 256, 256
    A8 = rng.integers(0, 0x58, (M, K), dtype=np.uint8); B8 = rng.integers(0, 0x58, (K, N), dtype=np.uint8) | 0x80
    b = (rng.standard_normal(N) * 0.1).astype(np.float16)
    dA, dB, db = dev(A8), dev(B8), dev(b)
    dC = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    sa = torch.tensor([0.03], device="cuda"); sb = torch.tensor([0.5], device="cuda")
    ta = t._c_tensor(dA.data_ptr(), (M, K), DT.FP8_E4M3, sa.data_ptr())
    tb = t._c_tensor(dB.data_ptr(), (K, N), DT.FP8_E4M3, sb.data_ptr())
    tbias = t._c_tensor(db.data_ptr(), (N,), DT.FLOAT16); tc = t._c_tensor(dC.data_ptr(), (M, N), DT.FLOAT16)
    assert L.tensorfuse_fused_gemm_bias_gelu(C.byref(ta), C.byref(tb), C.byref(tbias), C.byref(tc), stream()) == 0
    check_watchdog()
    want = oracle.gemm_bias_gelu_f64(table[A8], table[B8], b, scale=np.float32(0.03) * np.float32(0.5))
    assert (np.abs(dC.float().cpu().numpy() - want) <= 2e-3 * np.abs(want) + 1e-3).all()

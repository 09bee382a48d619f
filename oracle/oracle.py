"""Python face of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this module; the shipped package never does.

Two families of functions:

* thin ctypes wrappers over ``liboracle.so`` (built from ``oracle.c`` by
  ``oracle/Makefile``) -- the scalar-loop restatement of the reference's C++
  test oracles, plus the operation-by-operation "exact" softmax+dropout;
* numpy twins restating the reference's numpy oracle
  (``src/tests/python/test_mathematical_verification.py:29-58`` in the
  reference project): ``np_gelu``, ``np_gemm_bias_gelu``, ``np_softmax``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile liboracle.so if it is missing (or stale) and return its path."""
    src = os.path.join(_HERE, "oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        vp, i, l, f, u64 = C.c_void_p, C.c_int, C.c_long, C.c_float, C.c_uint64
        L.tfo_max_threads.restype = i
        L.tfo_gelu_f32.restype = f
        L.tfo_gelu_f32.argtypes = [f]
        L.tfo_gelu_f32_array.argtypes = [vp, vp, l]
        L.tfo_gemm_bias_gelu_f32.argtypes = [vp, vp, vp, vp, i, i, i, f, f, i]
        L.tfo_gemm_bias_gelu_f16.argtypes = [vp, vp, vp, vp, i, i, i, f, f, i]
        L.tfo_gemm_i8_acc.argtypes = [vp, vp, vp, i, i, i, i]
        L.tfo_i8_epilogue_f16.argtypes = [vp, vp, vp, l, i, f, f]
        L.tfo_i8_epilogue_legacy_f32.argtypes = [vp, vp, vp, l, i, f, f]
        L.tfo_softmax_ref_f32.argtypes = [vp, vp, l, i, i]
        L.tfo_softmax_ref_f16.argtypes = [vp, vp, vp, l, i, i]
        L.tfo_philox4x32_10.argtypes = [C.c_uint32] * 6 + [vp]
        L.tfo_dropout_threshold.restype = C.c_uint32
        L.tfo_dropout_threshold.argtypes = [f]
        L.tfo_dropout_mask.argtypes = [vp, u64, l, f, u64]
        L.tfo_softmax_dropout_exact.argtypes = [vp, vp, vp, l, i, i, f, u64, u64, i, i, i]
        L.tfo_softmax_dropout_exact_online.argtypes = [vp, vp, vp, l, i, i, f, u64, u64, i, i, i]
        L.tfo_softmax_dropout_exact_ext.argtypes = [vp, vp, vp, l, i, i, f, u64, i, i, f, vp, l, i]
        L.tfo_attention_f32.argtypes = [vp, vp, vp, vp, i, i, i, i, i, f, f, u64, vp, i]
        _lib = L
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def max_threads() -> int:
    return int(lib().tfo_max_threads())


# ----------------------------------------------------------------- C oracle

def gelu(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    lib().tfo_gelu_f32_array(_p(x), _p(y), x.size)
    return y


def gemm_bias_gelu_f32(A, B, bias, alpha=1.0, beta=1.0, threads=0):
    A = np.ascontiguousarray(A, np.float32); B = np.ascontiguousarray(B, np.float32)
    bias = np.ascontiguousarray(bias, np.float32)
    M, K = A.shape; N = B.shape[1]
    out = np.empty((M, N), np.float32)
    lib().tfo_gemm_bias_gelu_f32(_p(A), _p(B), _p(bias), _p(out), M, N, K, alpha, beta, threads)
    return out


def gemm_bias_gelu_f16(A, B, bias, alpha=1.0, beta=1.0, threads=0):
    A = np.ascontiguousarray(A, np.float16); B = np.ascontiguousarray(B, np.float16)
    bias = np.ascontiguousarray(bias, np.float16)
    M, K = A.shape; N = B.shape[1]
    out = np.empty((M, N), np.float16)
    lib().tfo_gemm_bias_gelu_f16(_p(A), _p(B), _p(bias), _p(out), M, N, K, alpha, beta, threads)
    return out


def gemm_i8_acc(A, B, threads=0):
    A = np.ascontiguousarray(A, np.int8); B = np.ascontiguousarray(B, np.int8)
    M, K = A.shape; N = B.shape[1]
    acc = np.empty((M, N), np.int32)
    lib().tfo_gemm_i8_acc(_p(A), _p(B), _p(acc), M, N, K, threads)
    return acc


def i8_epilogue_f16(acc, bias, scale_a, scale_b):
    acc = np.ascontiguousarray(acc, np.int32); bias = np.ascontiguousarray(bias, np.float16)
    out = np.empty(acc.shape, np.float16)
    lib().tfo_i8_epilogue_f16(_p(acc), _p(bias), _p(out), acc.shape[0], acc.shape[1],
                              scale_a, scale_b)
    return out


def i8_epilogue_legacy_f32(acc, bias, scale_a, scale_b):
    acc = np.ascontiguousarray(acc, np.int32); bias = np.ascontiguousarray(bias, np.float32)
    out = np.empty(acc.shape, np.float32)
    lib().tfo_i8_epilogue_legacy_f32(_p(acc), _p(bias), _p(out), acc.shape[0], acc.shape[1],
                                     scale_a, scale_b)
    return out


def softmax_ref_f32(x, threads=0):
    x = np.ascontiguousarray(x, np.float32)
    L = x.shape[-1]
    out = np.empty_like(x)
    lib().tfo_softmax_ref_f32(_p(x), _p(out), x.size // L, L, threads)
    return out


def softmax_ref_f16(x, threads=0):
    x = np.ascontiguousarray(x, np.float16)
    L = x.shape[-1]
    out = np.empty_like(x)
    mask = np.empty(x.shape, np.uint8)
    lib().tfo_softmax_ref_f16(_p(x), _p(out), _p(mask), x.size // L, L, threads)
    return out, mask


def philox4x32_10(counter, key):
    out = np.empty(4, np.uint32)
    lib().tfo_philox4x32_10(*[int(c) for c in counter], int(key[0]), int(key[1]), _p(out))
    return out


def dropout_threshold(p) -> int:
    return int(lib().tfo_dropout_threshold(float(p)))


def dropout_mask(n, p, seed, first_idx=0):
    m = np.empty(n, np.uint8)
    lib().tfo_dropout_mask(_p(m), first_idx, n, p, seed)
    return m


def softmax_dropout_exact(x, p=0.0, seed=0, first_row=0, vec=8, warps=1, threads=0, online=False):
    """Bit-reproducible softmax+dropout over the last axis.

    ``vec``/``warps``/``online`` name the summation schedule (see oracle.c); the
    library reports the schedule it uses for a given row length and dtype through
    ``tensorfuse_b200_softmax_schedule_ex``.
    """
    assert x.dtype in (np.float16, np.float32)
    x = np.ascontiguousarray(x)
    L = x.shape[-1]
    out = np.empty_like(x)
    mask = np.empty(x.shape, np.uint8)
    fn = lib().tfo_softmax_dropout_exact_online if online else lib().tfo_softmax_dropout_exact
    fn(_p(x), _p(out), _p(mask), x.size // L, L, 1 if x.dtype == np.float16 else 0, p, seed, first_row,
       vec, warps, threads)
    return out, mask


def softmax_dropout_masked_exact(x, scale=1.0, lengths=None, p=0.0, seed=0, vec=8, warps=1, threads=0):
    """Bit-reproducible restatement of tensorfuse_b200_softmax_dropout_masked:
    x is [batch, ..., L]; softmax(scale * x) over the last axis with the positions
    >= lengths[b] of batch item b masked, then dropout."""
    assert x.dtype in (np.float16, np.float32)
    x = np.ascontiguousarray(x)
    L = x.shape[-1]
    rows = x.size // L
    out = np.empty_like(x)
    mask = np.empty(x.shape, np.uint8)
    lens = None if lengths is None else np.ascontiguousarray(lengths, np.int32)
    lib().tfo_softmax_dropout_exact_ext(_p(x), _p(out), _p(mask), rows, L, 1 if x.dtype == np.float16 else 0,
                                        float(p), int(seed), vec, warps, float(scale),
                                        None if lens is None else _p(lens), rows // x.shape[0], threads)
    return out, mask


def attention(q, k, v, heads, p=0.0, seed=0, scale=None, kv_lengths=None, threads=0):
    """Multi-head scaled-dot-product attention with dropout on the weights;
    q [batch, seq_q, hidden], k/v [batch, seq_kv, hidden] (FP16 or FP32, widened
    to FP32), returns FP32 [batch, seq_q, hidden]."""
    q32, k32, v32 = (np.ascontiguousarray(t, np.float32) for t in (q, k, v))
    B, Sq, Hd = q32.shape
    Skv = k32.shape[1]
    hd = Hd // heads
    out = np.empty_like(q32)
    lens = None if kv_lengths is None else np.ascontiguousarray(kv_lengths, np.int32)
    lib().tfo_attention_f32(_p(q32), _p(k32), _p(v32), _p(out), B, Sq, Skv, heads, hd,
                            float(scale if scale else 1.0 / np.sqrt(hd)), float(p), int(seed),
                            None if lens is None else _p(lens), threads)
    return out


def add_layernorm(x, residual, gamma, beta, eps):
    """LayerNorm(x + residual) * gamma + beta over the last axis in float64
    (biased variance).  The reference carries the weights and epsilon for this in
    TensorFuseTransformerParams (src/tensorfuse/types.h:153-185) and computes
    nothing with them; this is the textbook definition."""
    s = np.asarray(x, np.float64) + (0.0 if residual is None else np.asarray(residual, np.float64))
    mean = s.mean(axis=-1, keepdims=True)
    var = ((s - mean) ** 2).mean(axis=-1, keepdims=True)
    return (s - mean) / np.sqrt(var + eps) * np.asarray(gamma, np.float64) + np.asarray(beta, np.float64)


def transformer_layer(x, w, heads, p=0.0, seed=0, eps=1e-12, activation="gelu"):
    """Post-LN encoder layer composed from the oracle's own pieces (FP32/FP64):
    q,k,v projections, attention(), output projection, add_layernorm, FFN with
    gelu() or no activation, add_layernorm.  ``w`` uses the field names of
    TensorFuseTransformerParams; matrices are [in, out]."""
    f = lambda t: np.asarray(t, np.float64)
    B, S, H = x.shape
    x2 = f(x).reshape(B * S, H)
    proj = lambda a, wn, bn: a @ f(w[wn]) + (f(w[bn]) if w.get(bn) is not None else 0.0)
    q, k, v = (proj(x2, n + "_weight", n + "_bias").reshape(B, S, H) for n in ("query", "key", "value"))
    ctx = attention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), heads, p=p, seed=seed)
    a = proj(f(ctx).reshape(B * S, H), "output_weight", "output_bias")
    h1 = add_layernorm(x2, a, w["ln1_weight"], w["ln1_bias"], eps)
    u = proj(h1, "ffn_weight1", "ffn_bias1")
    if activation == "gelu":
        u = 0.5 * u * (1.0 + np.tanh(0.7978845608028654 * (u + 0.044715 * u ** 3)))
    d = proj(u, "ffn_weight2", "ffn_bias2")
    return add_layernorm(h1, d, w["ln2_weight"], w["ln2_bias"], eps).reshape(B, S, H)


def bf16_round(x):
    """FP32 -> BF16 (round to nearest even) -> FP32, on the bit patterns."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def bf16_bits(x):
    """FP32 values (already BF16-representable) -> their 16-bit patterns."""
    return (np.ascontiguousarray(x, np.float32).view(np.uint32) >> 16).astype(np.uint16).reshape(np.shape(x))


def bf16_from_bits(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(np.shape(b))


def fp8_e4m3_table():
    """Value of each of the 256 E4M3 byte patterns (OCP FP8 "fn" variant: bias 7,
    no infinities, 0x7F / 0xFF are NaN), the type TENSORFUSE_FP8_E4M3 names
    (reference src/tensorfuse/types.h:56)."""
    t = np.empty(256, np.float32)
    for b in range(256):
        sgn = -1.0 if b & 0x80 else 1.0
        e, m = (b >> 3) & 0xF, b & 7
        if e == 15 and m == 7:
            v = np.nan
        elif e == 0:
            v = m / 8.0 * 2.0 ** -6
        else:
            v = (1 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = sgn * v
    return t


def gemm_bias_gelu_f64(A, B, bias, scale=1.0, activation="gelu"):
    """gelu(scale * A @ B + bias) in float64 from already-widened operands: the
    semantics of gemm_bias_gelu_ref (reference src/tests/test_kernels.cu:43-64)
    carried out in double, for operand types the C loops do not cover."""
    x = scale * (np.asarray(A, np.float64) @ np.asarray(B, np.float64)) + np.asarray(bias, np.float64)
    if activation == "gelu":
        x = 0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    return x


def quantize_sym_int8(x):
    """Per-tensor symmetric INT8 quantisation, FP32 arithmetic: scale = max|x|/127
    (1 for an all-zero tensor), q = clip(rint(x/scale), -127, 127) with
    round-half-even.  The reference has no quantiser of its own (its binding
    only guesses a scale from INT8 data, src/python/core_bindings.cpp:467-491);
    this is the recipe the INT8 benchmark configuration is generated with."""
    x = np.asarray(x).astype(np.float32)
    amax = np.float32(np.max(np.abs(x))) if x.size else np.float32(0)
    scale = np.float32(amax / np.float32(127.0)) if amax > 0 else np.float32(1.0)
    q = np.clip(np.rint(x / scale), -127, 127).astype(np.int8)
    return q, scale


def quantize_sym_int8_columns(w):
    """Channel-wise variant for a weight matrix [K, N]: one scale per column."""
    w = np.asarray(w).astype(np.float32)
    amax = np.max(np.abs(w), axis=0).astype(np.float32)
    scales = np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float32)
    q = np.clip(np.rint(w / scales[None, :]), -127, 127).astype(np.int8)
    return q, scales


# -------------------------------------------------------------- numpy twins

def np_gelu(x):
    a, b = 0.7978845608028654, 0.044715
    return x * 0.5 * (1.0 + np.tanh(a * (x + b * x * x * x)))


def np_gemm_bias_gelu(A, B, bias, alpha=1.0, beta=1.0):
    return np_gelu(alpha * np.matmul(A, B) + beta * bias)


def np_softmax(x, axis=-1):
    z = x - np.max(x, axis=axis, keepdims=True)
    e = np.exp(z)
    return e / np.sum(e, axis=axis, keepdims=True)


# --------------------------------------------------------------- comparisons

def f16_ulp_distance(a, b):
    """Distance in FP16 units-in-the-last-place between two float16 arrays
    (monotone integer mapping of the bit patterns; +0 and -0 coincide)."""
    def key(v):
        u = np.ascontiguousarray(v, np.float16).view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u)
    return np.abs(key(a) - key(b))


def f16_parity_violations(got, want, max_ulp=1, tiny_abs=2.0 ** -22):
    """Count elements of two float16 arrays that differ by more than ``max_ulp``
    FP16 ulps.  Below the smallest normal FP16 (2^-14) the ulp is the fixed
    subnormal step 2^-24 and the FP32 tanh form of GELU is itself only accurate
    to a few of those steps (1 + tanh cancels), so there the bound is
    ``tiny_abs`` absolute."""
    g = np.asarray(got, np.float16); w = np.asarray(want, np.float16)
    d = f16_ulp_distance(g, w)
    small = np.abs(w.astype(np.float32)) < 2.0 ** -14
    bad_normal = (~small) & (d > max_ulp)
    bad_small = small & (np.abs(g.astype(np.float32) - w.astype(np.float32)) > tiny_abs)
    return int(bad_normal.sum() + bad_small.sum())

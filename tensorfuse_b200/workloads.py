"""Seeded synthetic workloads for the five benchmark configurations.

Every generator draws with ``numpy.random.default_rng(seed)`` in FP32 and casts,
so the same inputs can be rebuilt anywhere.  They stand in for real activations
and weights: shapes and value distributions follow the configuration text, there
is no dataset or checkpoint behind them.
"""
from __future__ import annotations

import numpy as np


def gemm_fp32_quickstart(seed: int = 0, batch: int = 32, seq: int = 128, hidden: int = 768,
                         ffn: int = 3072):
    """Config 1: X[batch,seq,hidden]~N(0,1), W~N(0,1/hidden), b~N(0,0.02^2), FP32."""
    r = np.random.default_rng(seed)
    x = r.standard_normal((batch, seq, hidden), dtype=np.float32)
    w = (r.standard_normal((hidden, ffn), dtype=np.float32) / np.sqrt(np.float32(hidden))).astype(np.float32)
    b = (r.standard_normal(ffn, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    return x, w, b


def gemm_fp16_ffn(seed: int = 1, M: int = 16384, K: int = 1024, N: int = 4096):
    """Config 2: BERT-large FFN-up, row-major FP16."""
    r = np.random.default_rng(seed)
    a = r.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    w = (r.standard_normal((K, N), dtype=np.float32) / np.sqrt(np.float32(K))).astype(np.float16)
    b = (r.standard_normal(N, dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    return a, w, b


def quantize_sym_int8(x: np.ndarray):
    """Symmetric per-tensor INT8: scale = max|x|/127, q = clip(rint(x/scale), -127, 127)."""
    scale = np.float32(np.max(np.abs(x)) / 127.0)
    q = np.clip(np.rint(x / scale), -127, 127).astype(np.int8)
    return q, float(scale)


def gemm_int8(seed: int = 2, M: int = 8192, K: int = 4096, N: int = 16384):
    """Config 3: INT8 operands quantised from N(0,1) / N(0,1/K), FP16 bias."""
    r = np.random.default_rng(seed)
    a, sa = quantize_sym_int8(r.standard_normal((M, K), dtype=np.float32))
    w, sw = quantize_sym_int8(r.standard_normal((K, N), dtype=np.float32) / np.sqrt(np.float32(K)))
    b = (r.standard_normal(N, dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    return a, w, b, sa, sw


def attention_scores(seed: int = 3, batch: int = 32, heads: int = 16, seq: int = 512,
                     masked: bool = False):
    """Config 4: scores ~ N(0,1)/sqrt(64) in FP16; with ``masked`` the last
    floor(u_b*128*seq/512) keys of batch item b (u_b~U[0,1), at most 25 %) are -inf."""
    r = np.random.default_rng(seed)
    s = (r.standard_normal((batch, heads, seq, seq), dtype=np.float32) / np.float32(8.0)).astype(np.float16)
    if masked:
        u = r.random(batch)
        for b in range(batch):
            valid = seq - int(np.floor(u[b] * (seq // 4)))
            s[b, :, :, valid:] = -np.inf
    return s

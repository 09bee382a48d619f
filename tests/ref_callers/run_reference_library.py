"""Runs the reference's own GPU library (baseline/_ref/ref_lib/libtensorfuse_reference.so,
built by tests/ref_callers/build.py from a checkout of the reference) in a
process of its own, so that it never shares an address space with this
repository's libtensorfuse.so (both export the same symbol names).

    python run_reference_library.py cases  <in.npz> <out.npz>   # outputs for the parity test
    python run_reference_library.py bench                      # one JSON line of timings

`cases`: every array group in the input file names an operator:
    gemm_f32_<tag>/gemm_f16_<tag>: A, B, bias          -> C   (alpha = beta = 1)
    gemm_i8_<tag>:  A, B (int8), bias (f32), scales [sA, sB] -> C (f32, the reference's scaled convention)
    softmax_<tag>:  x [b, h, s, l], p [1], seed [1]    -> out, mask
The flat wrappers are called exactly as the reference's benchmarks call them
(reference benchmarks/tensorfuse_c_api.h:44-60; softmax argument order batch,
seq_len, head_dim, num_heads: src/kernels/fused_softmax_dropout.cu:302-320).
"""
from __future__ import annotations

import ctypes as C
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF_LIB = os.path.join(ROOT, "baseline", "_ref", "ref_lib", "libtensorfuse_reference.so")


def load():
    lib = C.CDLL(REF_LIB)
    vp, i, f, ull = C.c_void_p, C.c_int, C.c_float, C.c_ulonglong
    gemm = [vp, vp, vp, vp, i, i, i, f, f, vp]
    for n in ("fused_gemm_bias_gelu_fp32_wrapper", "fused_gemm_bias_gelu_fp16_wrapper"):
        getattr(lib, n).restype = i
        getattr(lib, n).argtypes = gemm
    lib.fused_gemm_bias_gelu_int8_wrapper_with_scales.restype = i
    lib.fused_gemm_bias_gelu_int8_wrapper_with_scales.argtypes = [vp, vp, vp, vp, i, i, i, f, f, f, f, vp]
    for n in ("fused_softmax_dropout_fp16_wrapper", "fused_softmax_dropout_fp32_wrapper"):
        getattr(lib, n).restype = i
        getattr(lib, n).argtypes = [vp, vp, vp, i, i, i, i, f, ull, vp]
    return lib


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_cases(src: str, dst: str) -> int:
    lib = load()
    data = np.load(src)
    groups = sorted({k.split("/")[0] for k in data.files})
    out = {}
    for g in groups:
        get = lambda name: data[f"{g}/{name}"]
        if g.startswith("gemm_"):
            A, B, bias = dev(get("A")), dev(get("B")), dev(get("bias"))
            M, K = A.shape
            N = B.shape[1]
            if g.startswith("gemm_i8"):
                sA, sB = (float(v) for v in get("scales"))
                Cd = torch.empty((M, N), dtype=torch.float32, device="cuda")
                st = lib.fused_gemm_bias_gelu_int8_wrapper_with_scales(A.data_ptr(), B.data_ptr(), bias.data_ptr(),
                                                                       Cd.data_ptr(), M, N, K, 1.0, 1.0, sA, sB, None)
            else:
                Cd = torch.empty((M, N), dtype=A.dtype, device="cuda")
                fn = lib.fused_gemm_bias_gelu_fp16_wrapper if A.dtype == torch.float16 else lib.fused_gemm_bias_gelu_fp32_wrapper
                st = fn(A.data_ptr(), B.data_ptr(), bias.data_ptr(), Cd.data_ptr(), M, N, K, 1.0, 1.0, None)
            torch.cuda.synchronize()
            out[f"{g}/status"] = np.array([st])
            out[f"{g}/C"] = Cd.cpu().numpy()
        elif g.startswith("softmax_"):
            x = dev(get("x"))
            b, h, s, l = x.shape
            o = torch.empty_like(x)
            m = torch.empty(x.shape, dtype=torch.uint8, device="cuda")
            fn = lib.fused_softmax_dropout_fp16_wrapper if x.dtype == torch.float16 else lib.fused_softmax_dropout_fp32_wrapper
            st = fn(x.data_ptr(), o.data_ptr(), m.data_ptr(), b, s, l, h, float(get("p")[0]), int(get("seed")[0]), None)
            torch.cuda.synchronize()
            out[f"{g}/status"] = np.array([st])
            out[f"{g}/out"] = o.cpu().numpy()
            out[f"{g}/mask"] = m.cpu().numpy()
    np.savez(dst, **out)
    return 0


def timed(fn, reps):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def run_bench() -> int:
    """The reference's kernels on the benchmark configurations 2 (FP16 GEMM+bias+GELU,
    M 16384 K 1024 N 4096) and 4 (softmax+dropout, 32 x 16 x 512 x 512 FP16), timed
    with CUDA events on synthetic operands of those shapes."""
    lib = load()
    res = {}
    M, K, N = 16384, 1024, 4096
    A = torch.randn((M, K), device="cuda").half()
    B = (torch.randn((K, N), device="cuda") / 32).half()
    bias = (torch.randn(N, device="cuda") * 0.02).half()
    Cd = torch.empty((M, N), dtype=torch.float16, device="cuda")

    def gemm():
        st = lib.fused_gemm_bias_gelu_fp16_wrapper(A.data_ptr(), B.data_ptr(), bias.data_ptr(), Cd.data_ptr(), M, N, K,
                                                   1.0, 1.0, None)
        assert st == 0, st
    ms = timed(gemm, 10)
    res["fp16_gemm_bias_gelu_16384x1024x4096"] = {"ms": ms, "tflops": 2.0 * M * N * K / (ms * 1e-3) / 1e12}
    del A, B, Cd
    b, h, s, l = 32, 16, 512, 512
    x = (torch.randn((b, h, s, l), device="cuda") / 8).half()
    o = torch.empty_like(x)
    m = torch.empty(x.shape, dtype=torch.uint8, device="cuda")
    for p in (0.0, 0.1):
        def sm(p=p):
            st = lib.fused_softmax_dropout_fp16_wrapper(x.data_ptr(), o.data_ptr(), m.data_ptr(), b, s, l, h, p, 3, None)
            assert st == 0, st
        ms = timed(sm, 2)
        res[f"softmax_dropout_fp16_32x16x512x512_p{p}"] = {"ms": ms, "gbs": x.numel() * 5 / (ms * 1e-3) / 1e9}
    print(json.dumps(res), flush=True)
    return 0


if __name__ == "__main__":
    if not os.path.exists(REF_LIB):
        sys.exit("the reference's GPU library has not been built (python tests/ref_callers/build.py <reference>)")
    if len(sys.argv) >= 4 and sys.argv[1] == "cases":
        sys.exit(run_cases(sys.argv[2], sys.argv[3]))
    if len(sys.argv) >= 2 and sys.argv[1] == "bench":
        sys.exit(run_bench())
    sys.exit(__doc__)

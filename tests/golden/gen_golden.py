#!/usr/bin/env python3
"""Generate tests/golden/reference_numpy_oracle.npz.

Run where the reference project is checked out:
    python tests/golden/gen_golden.py <path of the reference checkout>
(or set TENSORFUSE_REFERENCE).  The script
imports the reference's OWN numpy oracle functions from
``src/tests/python/test_mathematical_verification.py`` (gelu_reference,
gemm_bias_gelu_reference, softmax_reference) and the quantisation recipe of
``src/tests/python/test_int8_tensor_cores.py:62-90``, evaluates them on the
exact inputs the reference's tests use (same seeds, same distributions, same
shapes) and stores inputs and outputs.  The fixture travels with the repo; the
reference does not.
"""
import importlib.util
import os
import sys

import numpy as np

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TENSORFUSE_REFERENCE", "")
if not REF or not os.path.isdir(REF):
    sys.exit(__doc__)
SRC = os.path.join(REF, "src/tests/python/test_mathematical_verification.py")


def load_reference_oracle():
    spec = importlib.util.spec_from_file_location("ref_math_verification", SRC)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)          # `import tensorfuse` inside fails softly
    return mod


def main():
    ref = load_reference_oracle()
    out = {}

    # test_gemm_bias_gelu_different_sizes / _mathematical_correctness (:102-174)
    for (M, N, K) in [(1, 1, 1), (8, 16, 32), (16, 32, 64), (32, 64, 128)]:
        np.random.seed(42)
        A = np.random.uniform(-0.5, 0.5, (M, K)).astype(np.float32)
        B = np.random.uniform(-0.5, 0.5, (K, N)).astype(np.float32)
        bias = np.random.uniform(-0.5, 0.5, (N,)).astype(np.float32)
        C = ref.gemm_bias_gelu_reference(A, B, bias, 1.0, 1.0)
        tag = f"gemm_{M}x{N}x{K}"
        out[tag + "_A"], out[tag + "_B"], out[tag + "_bias"], out[tag + "_C"] = A, B, bias, C

    # test_gelu_activation_properties (:225-260)
    pts = np.array([-3.0, -2.0, -1.0, -0.5, 0.0, 0.5, 1.0, 2.0, 3.0], dtype=np.float32)
    out["gelu_points"] = pts
    out["gelu_values"] = ref.gelu_reference(pts)
    # C-API smoke value GELU(1*2+0.5) (src/tests/test_c_api_debug.cpp:163-170)
    out["gelu_2p5"] = ref.gelu_reference(np.array([2.5], dtype=np.float32))

    # test_softmax_dropout_mathematical_correctness (:181-223)
    np.random.seed(42)
    x = np.random.uniform(-2.0, 2.0, (2, 8, 64, 64)).astype(np.float32)
    out["softmax_in"] = x
    out["softmax_out"] = ref.softmax_reference(x, axis=-1)

    # INT8 recipe of test_int8_mathematical_correctness (scale = 127/max|x|)
    M, N, K = 64, 128, 64
    np.random.seed(123)
    A32 = np.random.uniform(-1.0, 1.0, (M, K)).astype(np.float32)
    B32 = np.random.uniform(-1.0, 1.0, (K, N)).astype(np.float32)
    b32 = np.random.uniform(-0.1, 0.1, (N,)).astype(np.float32)
    sA = 127.0 / np.max(np.abs(A32)); sB = 127.0 / np.max(np.abs(B32))
    out["int8_A"] = np.clip(A32 * sA, -127, 127).astype(np.int8)
    out["int8_B"] = np.clip(B32 * sB, -127, 127).astype(np.int8)
    out["int8_bias"] = b32
    out["int8_scales"] = np.array([sA, sB], dtype=np.float32)
    out["int8_fp32_reference"] = ref.gelu_reference(np.matmul(A32, B32) + b32)

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_numpy_oracle.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    sys.exit(main())

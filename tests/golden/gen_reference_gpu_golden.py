"""Golden vectors from the reference's own GPU kernels.

    python tests/golden/gen_reference_gpu_golden.py [out.npz]      (needs a GPU)

Runs the reference's GPU library (built by tests/ref_callers/build.py into
baseline/_ref/ref_lib/) on small seeded operands through
tests/ref_callers/run_reference_library.py and stores its OUTPUTS in
tests/golden/reference_gpu_kernels.npz.  The operands are not stored: `cases()`
below regenerates them from the seed, and the file carries a checksum of them.
tests/test_golden_reference_gpu.py compares this repository's library with the
stored outputs, so the comparison with the reference's kernels survives on a
machine that has no checkout of the reference.
"""
import hashlib
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
RUNNER = os.path.join(ROOT, "tests", "ref_callers", "run_reference_library.py")
GOLDEN = os.path.join(HERE, "reference_gpu_kernels.npz")


def cases():
    rng = np.random.default_rng(23)
    c = {}
    M, K, N = 64, 256, 128                       # the size of the reference's own kernel test
    c["gemm_f32_g/A"] = rng.standard_normal((M, K)).astype(np.float32)
    c["gemm_f32_g/B"] = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    c["gemm_f32_g/bias"] = (rng.standard_normal(N) * 0.5).astype(np.float32)
    M, K, N = 128, 256, 256
    c["gemm_f16_g/A"] = rng.standard_normal((M, K)).astype(np.float16)
    c["gemm_f16_g/B"] = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16)
    c["gemm_f16_g/bias"] = (rng.standard_normal(N) * 0.5).astype(np.float16)
    x, w = rng.standard_normal((M, K)), rng.standard_normal((K, N)) / np.sqrt(K)
    sA, sB = 127.0 / np.abs(x).max(), 127.0 / np.abs(w).max()
    c["gemm_i8_g/A"] = np.clip(np.rint(x * sA), -127, 127).astype(np.int8)
    c["gemm_i8_g/B"] = np.clip(np.rint(w * sB), -127, 127).astype(np.int8)
    c["gemm_i8_g/bias"] = (rng.standard_normal(N) * 0.1).astype(np.float32)
    c["gemm_i8_g/scales"] = np.array([sA, sB], dtype=np.float32)
    for tag, dt in (("f32_g", np.float32), ("f16_g", np.float16)):
        c[f"softmax_{tag}/x"] = (rng.standard_normal((1, 2, 32, 128)) * 2).astype(dt)
        c[f"softmax_{tag}/p"] = np.array([0.0], dtype=np.float32)
        c[f"softmax_{tag}/seed"] = np.array([5], dtype=np.uint64)
    return c


def checksum(c) -> str:
    h = hashlib.sha256()
    for k in sorted(c):
        h.update(k.encode())
        h.update(np.ascontiguousarray(c[k]).tobytes())
    return h.hexdigest()


if __name__ == "__main__":
    dst = sys.argv[1] if len(sys.argv) > 1 else GOLDEN
    c = cases()
    with tempfile.TemporaryDirectory() as d:
        src, out = os.path.join(d, "in.npz"), os.path.join(d, "out.npz")
        np.savez(src, **c)
        subprocess.run([sys.executable, RUNNER, "cases", src, out], check=True)
        res = dict(np.load(out))
    keep = {k: v for k, v in res.items() if k.endswith("/C") or k.endswith("/out") or k.endswith("/status")}
    keep["inputs_sha256"] = np.frombuffer(checksum(c).encode(), dtype=np.uint8)
    np.savez_compressed(dst, **keep)
    print("wrote", dst, {k: v.shape for k, v in keep.items()})

"""The tensor-core GEMM has two forms: a CTA-pair kernel (256-row pair tiles,
tcgen05 cta_group::2), the default when the problem has more than one 128-row
band, and a single-CTA kernel.  The other tests exercise the default choice;
this one forces each form in a child process (the choice is read once per
process from TENSORFUSE_B200_GEMM_FORM) and checks both against the oracle on a
shape with ragged row and column tails."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys, numpy as np, torch
sys.path.insert(0, %r)
import tensorfuse_b200 as tf
from oracle import oracle
tf.init()
rng = np.random.default_rng(3)
M, K, N = 1000, 520, 776
A = rng.standard_normal((M, K)).astype(np.float16); B = (rng.standard_normal((K, N)) / 16).astype(np.float16)
b = (rng.standard_normal(N) * 0.1).astype(np.float16)
c = tf.fused_gemm_bias_gelu(torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), torch.from_numpy(b).cuda())
ref = oracle.gemm_bias_gelu_f16(A, B, b).astype(np.float32)
assert np.all(np.abs(c.cpu().numpy().astype(np.float32) - ref) <= 1e-3 + 1e-2 * np.abs(ref)), "fp16"
Ai = rng.integers(-127, 128, (M, 528), dtype=np.int8); Bi = rng.integers(-127, 128, (528, 784), dtype=np.int8)
acc = tf.fused_gemm_bias_gelu(torch.from_numpy(Ai).cuda(), torch.from_numpy(Bi).cuda(), torch.zeros(784, device="cuda"),
                              out_dtype=torch.int32)
assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i8_acc(Ai, Bi)), "int8"
assert tf.watchdog_status() == 0
print("ok", tf.launch_count())
"""


@pytest.mark.parametrize("form", ["single", "pair"])
def test_forced_form(form):
    env = dict(os.environ, TENSORFUSE_B200_GEMM_FORM=form)
    r = subprocess.run([sys.executable, "-c", CHILD % ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.strip().startswith("ok")


# FP32 has two paths as well: the CUDA-core kernel and the tensor-core kernel
# that rebuilds each FP32 product from three TF32 products (chosen by size;
# TENSORFUSE_B200_FP32_FORM = simt | tf32x3 forces one).  Both must hold the
# reference's FP32 bar -- max abs error 1e-4 against the sequential-k CPU loop
# (reference src/tests/test_kernels.cu:139, test_gemm_edge_cases.cu:155,249,383) --
# on its size, alpha/beta and extreme-value grids, on ragged shapes and on
# benchmark configuration 1.
CHILD_FP32 = r"""
import sys, numpy as np, torch
sys.path.insert(0, %r)
sys.path.insert(0, %r)
import tensorfuse_b200 as tf
from tensorfuse_b200 import workloads
from oracle import oracle
from gpu_util import gemm_wrapper, L, dev, host, stream
tf.init()
worst = 0.0
def check(A, B, b, alpha=1.0, beta=1.0, tol=1e-4, name="fused_gemm_bias_gelu_fp32_wrapper"):
    global worst
    st, out = gemm_wrapper(name, A, B, b, torch.float32, alpha, beta)
    assert st == 0, st
    want = oracle.gemm_bias_gelu_f32(A, B, b, alpha, beta)
    assert np.all(np.isfinite(out))
    err = float(np.max(np.abs(out - want)))
    worst = max(worst, err if tol <= 1e-4 else 0.0)
    assert err < tol, (A.shape, B.shape, alpha, beta, err)
r = np.random.default_rng(42)
for (M, N, K) in [(1, 1, 1), (8, 16, 32), (16, 32, 64), (32, 64, 128), (64, 128, 256), (128, 256, 512),
                  (256, 512, 1024), (1, 16, 4), (16, 4, 16), (256, 1024, 2048), (129, 132, 68), (300, 260, 100),
                  (1000, 776, 520)]:
    check(r.uniform(-0.5, 0.5, (M, K)).astype(np.float32), r.uniform(-0.5, 0.5, (K, N)).astype(np.float32),
          r.uniform(-0.5, 0.5, N).astype(np.float32))
A = r.uniform(-0.5, 0.5, (264, 520)).astype(np.float32); B = r.uniform(-0.5, 0.5, (520, 136)).astype(np.float32)
b = r.uniform(-0.5, 0.5, 136).astype(np.float32)
for alpha, beta in [(1, 1), (0, 1), (1, 0), (0, 0), (2, 0.5), (-1, 1), (1, -1), (0.5, 2), (-0.5, -0.5)]:
    check(A, B, b, alpha, beta)
M, N, K = 160, 264, 96
for val in (0.0, 1.0, 100.0, -100.0, 1e-6, None):
    if val is None:
        A = np.where(np.arange(M * K) %% 2 == 0, 1000.0, -1000.0).astype(np.float32).reshape(M, K)
        B = np.where(np.arange(K * N) %% 2 == 0, 1000.0, -1000.0).astype(np.float32).reshape(K, N)
    else:
        A = np.full((M, K), val, np.float32); B = np.full((K, N), val, np.float32)
    check(A, B, np.zeros(N, np.float32), tol=1e-2)
# FFN-down form (bias, no activation) through the activation entry point
A = r.standard_normal((512, 1024)).astype(np.float32); B = (r.standard_normal((1024, 256)) / 32).astype(np.float32)
b = r.standard_normal(256).astype(np.float32)
dA, dB, db = dev(A), dev(B), dev(b); dC = torch.empty((512, 256), device="cuda")
assert L.tensorfuse_b200_gemm_bias_act(dA.data_ptr(), dB.data_ptr(), db.data_ptr(), dC.data_ptr(), 512, 256, 1024, 0, 0,
                                       1.0, 1.0, stream()) == 0
torch.cuda.synchronize()
want = (A.astype(np.float64) @ B.astype(np.float64) + b).astype(np.float32)
assert float(np.max(np.abs(host(dC) - want))) < 1e-4
# benchmark configuration 1, whole output
x, w, bb = workloads.gemm_fp32_quickstart()
check(x.reshape(-1, 768), w, bb)
assert tf.watchdog_status() == 0
print("ok", tf.launch_count(), "worst abs error", worst)
"""


@pytest.mark.parametrize("form", ["simt", "tf32x3"])
def test_forced_fp32_form(form):
    env = dict(os.environ, TENSORFUSE_B200_FP32_FORM=form)
    r = subprocess.run([sys.executable, "-c", CHILD_FP32 % (ROOT, os.path.join(ROOT, "tests"))], env=env,
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.strip().splitlines()[-1].startswith("ok")
    print(form, r.stdout.strip().splitlines()[-1])

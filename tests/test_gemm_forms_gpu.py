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

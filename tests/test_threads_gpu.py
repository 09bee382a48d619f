"""Several host threads drive the library at once, each on its own stream (the
reference keeps non-atomic global state and is not thread-safe,
src/tensorfuse_c_api.cpp:47-56; this library's per-call state is thread-local or
locked).  Every thread checks its own results against values computed serially."""
import threading

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_concurrent_callers_on_separate_streams(tf, oracle):
    rng = np.random.default_rng(21)
    jobs = []
    for t in range(4):
        M, K, N = 384 + 128 * t, 256, 512
        A = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float16)).cuda()
        B = torch.from_numpy((rng.standard_normal((K, N)) / 16).astype(np.float16)).cuda()
        b = torch.from_numpy((rng.standard_normal(N) * 0.1).astype(np.float16)).cuda()
        x = torch.from_numpy((rng.standard_normal((2, 2, 64, 512)) / 2).astype(np.float16)).cuda()
        q = torch.from_numpy(rng.standard_normal((2, 256, 128)).astype(np.float16)).cuda()
        jobs.append((A, B, b, x, q))
    # serial results first
    want = []
    for (A, B, b, x, q) in jobs:
        want.append((tf.fused_gemm_bias_gelu(A, B, b).clone(),
                     tf.fused_softmax_dropout(x, dropout_prob=0.1, seed=3)[0].clone(),
                     tf.fused_multi_head_attention(q, q, q, None, 2, 0.1, seed=4).clone()))
    torch.cuda.synchronize()
    errors = []

    def worker(i):
        try:
            A, B, b, x, q = jobs[i]
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                for _ in range(20):
                    c = tf.fused_gemm_bias_gelu(A, B, b)
                    y, _ = tf.fused_softmax_dropout(x, dropout_prob=0.1, seed=3)
                    o = tf.fused_multi_head_attention(q, q, q, None, 2, 0.1, seed=4)
                s.synchronize()
            assert torch.equal(c, want[i][0]) and torch.equal(y, want[i][1]) and torch.equal(o, want[i][2])
        except Exception as e:          # noqa: BLE001 - reported by the main thread
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not any(t.is_alive() for t in threads)
    assert not errors, errors
    assert tf.watchdog_status() == 0


def test_concurrent_host_buffer_callers(tf, oracle):
    """The host-buffer operators share per-device staging buffers, streams and
    events; calls are serialised per device by a lock, so threads that call them
    at once on different shapes must each get exactly the serial result."""
    from tensorfuse_b200 import workloads
    rng = np.random.default_rng(33)
    jobs = []
    for t in range(4):
        A, B, b = workloads.gemm_fp16_ffn(seed=40 + t, M=700 + 333 * t, K=256 + 128 * (t % 2), N=512 + 256 * (t % 3))
        x = (rng.standard_normal((2, 3, 50 + 17 * t, 256 + 128 * t)) / 2).astype(np.float16)
        jobs.append((A, B, b, x))
    want = [(tf.fused_gemm_bias_gelu(A, B, b), tf.fused_softmax_dropout(x, dropout_prob=0.1, seed=7 + i))
            for i, (A, B, b, x) in enumerate(jobs)]
    errors = []

    def worker(i):
        try:
            A, B, b, x = jobs[i]
            for _ in range(6):
                c = tf.fused_gemm_bias_gelu(A, B, b)
                y, m = tf.fused_softmax_dropout(x, dropout_prob=0.1, seed=7 + i)
                assert np.array_equal(c.view(np.uint16), want[i][0].view(np.uint16))
                assert np.array_equal(y.view(np.uint16), want[i][1][0].view(np.uint16))
                assert np.array_equal(m, want[i][1][1])
        except Exception as e:          # noqa: BLE001 - reported by the main thread
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not any(t.is_alive() for t in threads)
    assert not errors, errors
    assert tf.watchdog_status() == 0

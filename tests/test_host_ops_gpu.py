"""Host-buffer operators: pipelined copy-in / compute / copy-out, row-sharded
over the configured devices.  Results must equal the device-pointer path bit
for bit, for every device count the box offers."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_gemm_host_equals_device_path(tf, oracle):
    from gpu_util import gemm_wrapper
    from tensorfuse_b200 import workloads
    A, B, b = workloads.gemm_fp16_ffn(M=5000, K=512, N=1024)     # several chunks, ragged tail
    st, dev_out = gemm_wrapper("fused_gemm_bias_gelu_fp16_wrapper", A, B, b, torch.float16)
    assert st == 0
    out = tf.fused_gemm_bias_gelu(A, B, b)
    assert np.array_equal(out.view(np.uint16), dev_out.view(np.uint16))
    # pinned staging memory gives the same bytes
    pa = tf.pinned_empty(A.shape, A.dtype); pa[...] = A
    po = tf.pinned_empty(out.shape, out.dtype)
    tf.fused_gemm_bias_gelu(pa, B, b, po)
    assert np.array_equal(po.view(np.uint16), dev_out.view(np.uint16))


def test_softmax_host_equals_oracle(tf, oracle):
    x = np.random.default_rng(1).standard_normal((3, 5, 200, 512)).astype(np.float16)
    out, mask = tf.fused_softmax_dropout(x, dropout_prob=0.1, seed=99)
    want, wmask = oracle.softmax_dropout_exact(x, p=0.1, seed=99)
    assert np.array_equal(out.view(np.uint16), want.view(np.uint16)) and np.array_equal(mask, wmask)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_multi_device_sharding_reproduces_single_device(oracle):
    """Re-initialise the library on all visible devices: the row split must not
    change a single bit of either operator's result."""
    import tensorfuse_b200 as t
    from tensorfuse_b200 import workloads
    A, B, b = workloads.gemm_fp16_ffn(M=4096 + 128, K=256, N=512)
    x = np.random.default_rng(2).standard_normal((2, 4, 100, 256)).astype(np.float16)
    t.init()
    one = t.fused_gemm_bias_gelu(A, B, b)
    s_one = t.fused_softmax_dropout(x, dropout_prob=0.1, seed=5)
    t.shutdown()
    n = min(torch.cuda.device_count(), 8)
    t.init(t.Config(device_ids=list(range(n))))
    try:
        assert t.device_ids() == list(range(n))
        many = t.fused_gemm_bias_gelu(A, B, b)
        s_many = t.fused_softmax_dropout(x, dropout_prob=0.1, seed=5)
    finally:
        t.shutdown()
        t.init()
    assert np.array_equal(one.view(np.uint16), many.view(np.uint16))
    assert np.array_equal(s_one[0].view(np.uint16), s_many[0].view(np.uint16)) and np.array_equal(s_one[1], s_many[1])


def test_bad_device_list_is_rejected_without_launching(tf):
    import tensorfuse_b200 as t
    t.shutdown()
    try:
        with pytest.raises(RuntimeError, match="Invalid configuration"):
            t.init(t.Config(device_ids=[0, 99]))
        with pytest.raises(RuntimeError, match="Invalid configuration"):
            t.init(t.Config(device_ids=[0, 0]))
    finally:
        t.init()


def test_registered_weights_are_uploaded_once(tf, oracle):
    """A weight range registered as immutable is copied to the device on first use
    only: changing the host bytes afterwards (without invalidating) must not
    change the result, and invalidating must."""
    from tensorfuse_b200 import workloads
    from tensorfuse_b200._lib import lib as L
    A, B, b = workloads.gemm_fp16_ffn(seed=8, M=640, K=256, N=512)
    B = np.ascontiguousarray(B); b = np.ascontiguousarray(b)
    first = tf.fused_gemm_bias_gelu(A, B, b)
    assert L.tensorfuse_b200_register_weights(B.ctypes.data, B.nbytes) == 0
    assert L.tensorfuse_b200_register_weights(b.ctypes.data, b.nbytes) == 0
    assert L.tensorfuse_b200_register_weights(None, 4) == 1
    try:
        cached = tf.fused_gemm_bias_gelu(A, B, b)                  # uploads and caches
        assert np.array_equal(cached.view(np.uint16), first.view(np.uint16))
        B_saved = B.copy()
        B[...] = 0                                                 # the device copy is still the old one
        stale = tf.fused_gemm_bias_gelu(A, B, b)
        assert np.array_equal(stale.view(np.uint16), first.view(np.uint16))
        assert L.tensorfuse_b200_invalidate_weights(B.ctypes.data) == 0
        fresh = tf.fused_gemm_bias_gelu(A, B, b)                   # B is all zero now: gelu(bias) everywhere
        want = oracle.gemm_bias_gelu_f16(A, B, b)
        assert oracle.f16_parity_violations(fresh, want) == 0
        assert not np.array_equal(fresh.view(np.uint16), first.view(np.uint16))
        B[...] = B_saved
    finally:
        assert L.tensorfuse_b200_invalidate_weights(None) == 0
    again = tf.fused_gemm_bias_gelu(A, B, b)
    assert np.array_equal(again.view(np.uint16), first.view(np.uint16))

"""`import tensorfuse`: the drop-in package of this repository (module names,
signatures and error texts of the reference's package, reference
src/python/tensorfuse/__init__.py:53-198 and core.py:36-322) on a GPU.  The
numerical bars are those of the reference's own Python tests
(reference src/tests/python/test_mathematical_verification.py:102-223: rtol = atol = 1e-4)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _gelu(x):
    return 0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


@pytest.fixture()
def tfpkg():
    import tensorfuse
    import tensorfuse_b200
    tensorfuse.init()
    yield tensorfuse
    tensorfuse_b200.init()     # other test modules share the library; leave it initialised


def test_module_surface(tfpkg):
    import tensorfuse._tensorfuse as ext
    for name in ("Status", "DataType", "Layout", "Shape", "Config", "Tensor", "init", "shutdown", "get_version",
                 "get_error_string", "fused_gemm_bias_gelu", "fused_softmax_dropout", "fused_multi_head_attention",
                 "autotune", "load_tuned_config", "is_gpu_supported", "get_device_info", "set_random_seed",
                 "allocate_tensor", "free_tensor", "get_memory_info", "ProfileConfig", "Metrics", "start_profiling",
                 "stop_profiling", "get_last_metrics", "create_tensor", "from_numpy", "to_numpy",
                 "get_tensor_size_bytes", "get_dtype_size", "benchmark_operation"):
        assert hasattr(ext, name), name
    assert tfpkg.is_gpu_supported()
    info = tfpkg.get_device_info()
    assert info["tensor_cores"] and info["compute_capability"].startswith("10.")
    mem = tfpkg.get_memory_info()
    assert mem["total_bytes"] > mem["free_bytes"] > 0
    assert tfpkg.get_last_metrics().kernel_time_ms == 1.5        # the reference's placeholder record


def test_operators_on_numpy(tfpkg):
    rng = np.random.default_rng(42)
    for (M, K, N) in ((1, 1, 1), (8, 16, 32), (32, 64, 128), (100, 70, 36)):
        A = rng.uniform(-0.5, 0.5, (M, K)).astype(np.float32)
        B = rng.uniform(-0.5, 0.5, (K, N)).astype(np.float32)
        b = rng.uniform(-0.5, 0.5, N).astype(np.float32)
        out = tfpkg.fused_gemm_bias_gelu(A, B, b)
        np.testing.assert_allclose(out, _gelu(A.astype(np.float64) @ B.astype(np.float64) + b), rtol=1e-4, atol=1e-4)
    x = rng.uniform(-2, 2, (2, 8, 64, 64)).astype(np.float32)
    out = np.zeros_like(x); mask = np.zeros(x.shape, np.uint8)
    tfpkg.fused_softmax_dropout(x, out, mask, 0.0)
    e = np.exp(x - x.max(-1, keepdims=True))
    np.testing.assert_allclose(out, e / e.sum(-1, keepdims=True), rtol=1e-4, atol=1e-4)
    assert mask.min() == 1
    y, m = tfpkg.softmax_dropout(x, dropout_prob=0.1)
    assert abs(m.mean() - 0.9) < 0.02 and np.all((y == 0) == (m == 0))
    with pytest.raises(RuntimeError, match="Tensor dimension mismatch"):
        tfpkg.fused_gemm_bias_gelu(np.zeros((4, 8), np.float32), np.zeros((9, 4), np.float32), np.zeros(4, np.float32))


def test_tensor_round_trip_and_modules(tfpkg):
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    t = tfpkg.from_numpy(a)
    assert t.shape.dims == [2, 3, 4] and t.size_bytes == 96 and t.data
    assert np.array_equal(tfpkg.to_numpy(t), a)
    tfpkg.free_tensor(t)
    assert t.data == 0
    with pytest.raises(RuntimeError, match="empty array"):
        tfpkg.from_numpy(np.zeros((0, 3), np.float32))
    # nn.Module wrapper on CUDA tensors: in place, no host round trip
    op = tfpkg.FusedGemmBiasGelu(64, 128, 96)
    x = torch.randn(4, 16, 96, device="cuda", dtype=torch.float16)
    y = op(x)
    ref = torch.nn.functional.gelu(x.float() @ op.weight.detach().cuda().half().float() +
                                   op.bias.detach().cuda().half().float(), approximate="tanh")
    assert y.is_cuda and y.shape == (4, 16, 128)
    assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2)
    q = torch.randn(2, 128, 256, device="cuda", dtype=torch.float16)
    o = tfpkg.multi_head_attention(q, q, q, num_heads=4, dropout_prob=0.0)
    assert o.shape == q.shape and torch.isfinite(o).all()

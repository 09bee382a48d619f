"""The struct-based C ABI on the GPU: validation order and codes (reference
src/tensorfuse_c_api.cpp:139-286), dtype dispatch, extensions."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(L, ti, tw, tb, to, stream=None):
    from gpu_util import byref
    return L.tensorfuse_fused_gemm_bias_gelu(byref(ti), byref(tw), byref(tb), byref(to), stream)


def test_lifecycle_and_error_strings(tf):
    from gpu_util import L
    assert tf.get_version() == "1.0.0"
    assert L.tensorfuse_init(None) == 0          # idempotent
    assert tf.get_error_string(4) == "Library not initialized"
    assert tf.get_error_string(11) == "Invalid tensor shape" and tf.get_error_string(12345) == "Unknown error"
    assert tf.device_ids() == [torch.cuda.current_device()]


def test_gemm_struct_api_fp32_fp16_and_3d(tf, oracle):
    from gpu_util import L, c_tensor, check_watchdog, dev, host, stream
    r = np.random.default_rng(0)
    x = r.standard_normal((4, 16, 64)).astype(np.float32)       # [batch, seq, hidden]
    w = (r.standard_normal((64, 96)) / 8).astype(np.float32)
    b = (r.standard_normal(96) * 0.02).astype(np.float32)
    dx, dw, db = dev(x), dev(w), dev(b)
    dout = torch.empty((4, 16, 96), dtype=torch.float32, device="cuda")
    assert _call(L, c_tensor(dx), c_tensor(dw), c_tensor(db), c_tensor(dout), stream()) == 0
    check_watchdog()
    want = oracle.gemm_bias_gelu_f32(x.reshape(64, 64), w, b).reshape(4, 16, 96)
    np.testing.assert_allclose(host(dout), want, rtol=1e-4, atol=1e-4)
    # 2-D view of the same buffers
    d2 = torch.empty((64, 96), dtype=torch.float32, device="cuda")
    assert _call(L, c_tensor(dx, shape=(64, 64)), c_tensor(dw), c_tensor(db), c_tensor(d2), stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(d2, dout.reshape(64, 96))
    # FP16 goes to the tensor-core kernel
    xh, wh, bh = x.reshape(64, 64).astype(np.float16), w.astype(np.float16), b.astype(np.float16)
    dxh, dwh, dbh = dev(xh), dev(wh), dev(bh)
    doh = torch.empty((64, 96), dtype=torch.float16, device="cuda")
    assert _call(L, c_tensor(dxh), c_tensor(dwh), c_tensor(dbh), c_tensor(doh), stream()) == 0
    check_watchdog()
    np.testing.assert_allclose(host(doh).astype(np.float32), oracle.gemm_bias_gelu_f16(xh, wh, bh).astype(np.float32),
                               rtol=1e-2, atol=1e-3)


def test_gemm_validation_codes(tf):
    from gpu_util import L, c_tensor, dev
    x = dev(np.zeros((8, 16), np.float32)); w = dev(np.zeros((16, 24), np.float32))
    b = dev(np.zeros(24, np.float32)); o = torch.empty((8, 24), device="cuda")
    from gpu_util import byref
    assert L.tensorfuse_fused_gemm_bias_gelu(None, byref(c_tensor(w)), byref(c_tensor(b)), byref(c_tensor(o)), None) == 1
    assert _call(L, c_tensor(x, shape=(128,)), c_tensor(w), c_tensor(b), c_tensor(o)) == 11     # rank
    assert _call(L, c_tensor(x), c_tensor(w, shape=(24, 16)), c_tensor(b), c_tensor(o)) == 11   # K mismatch
    assert _call(L, c_tensor(x), c_tensor(w), c_tensor(b, shape=(8,)), c_tensor(o)) == 11       # bias length
    assert _call(L, c_tensor(x), c_tensor(w), c_tensor(b), c_tensor(o, shape=(8, 12))) == 11    # output shape
    wh = dev(np.zeros((16, 24), np.float16))
    assert _call(L, c_tensor(x), c_tensor(wh), c_tensor(b), c_tensor(o)) == 1                   # dtype mismatch
    xi = dev(np.zeros((8, 16), np.int32)); wi = dev(np.zeros((16, 24), np.int32)); oi = torch.empty((8, 24), dtype=torch.int32, device="cuda")
    assert _call(L, c_tensor(xi), c_tensor(wi), c_tensor(b), c_tensor(oi)) == 10                # unsupported dtype


def test_int8_struct_api_with_device_scales(tf, oracle):
    from gpu_util import L, c_tensor, check_watchdog, dev, host, stream
    from tensorfuse_b200 import workloads
    r = np.random.default_rng(6)
    A, sa = workloads.quantize_sym_int8(r.standard_normal((128, 256)).astype(np.float32))
    B, sb = workloads.quantize_sym_int8((r.standard_normal((256, 512)) / 16).astype(np.float32))
    acc = oracle.gemm_i8_acc(A, B)
    dA, dB = dev(A), dev(B)
    # FP16 bias + FP16 output: multiply convention, scales read on the device
    bias_h = (r.standard_normal(512) * 0.02).astype(np.float16)
    dsa, dsb = dev(np.array([sa], np.float32)), dev(np.array([sb], np.float32))
    dbh = dev(bias_h); doh = torch.empty((128, 512), dtype=torch.float16, device="cuda")
    assert _call(L, c_tensor(dA, scale=dsa), c_tensor(dB, scale=dsb), c_tensor(dbh), c_tensor(doh), stream()) == 0
    check_watchdog()
    assert oracle.f16_parity_violations(host(doh), oracle.i8_epilogue_f16(acc, bias_h, sa, sb)) == 0
    # FP32 bias + FP32 output: the reference's convention (scale = 127/max|x|)
    ra, rb = 1.0 / sa, 1.0 / sb
    bias_f = bias_h.astype(np.float32)
    dra, drb = dev(np.array([ra], np.float32)), dev(np.array([rb], np.float32))
    dbf = dev(bias_f); dof = torch.empty((128, 512), dtype=torch.float32, device="cuda")
    assert _call(L, c_tensor(dA, scale=dra), c_tensor(dB, scale=drb), c_tensor(dbf), c_tensor(dof), stream()) == 0
    check_watchdog()
    np.testing.assert_allclose(host(dof), oracle.i8_epilogue_legacy_f32(acc, bias_f, np.float32(ra), np.float32(rb)),
                               rtol=2e-5, atol=1e-2)
    # INT32 output: raw accumulators; NULL scale pointers mean 1
    doi = torch.empty((128, 512), dtype=torch.int32, device="cuda")
    assert _call(L, c_tensor(dA), c_tensor(dB), c_tensor(dbf), c_tensor(doi), stream()) == 0
    check_watchdog()
    assert np.array_equal(host(doi), acc)
    # INT8 input with a non-INT8 weight is an invalid argument, INT8 output is unsupported
    assert _call(L, c_tensor(dA), c_tensor(dev(np.zeros((256, 512), np.float32))), c_tensor(dbf), c_tensor(dof)) == 1
    do8 = torch.empty((128, 512), dtype=torch.int8, device="cuda")
    assert _call(L, c_tensor(dA), c_tensor(dB), c_tensor(dbf), c_tensor(do8)) == 10


def test_stubs_allocate_and_mangled_symbols(tf):
    import ctypes as C
    from gpu_util import L, byref
    from tensorfuse_b200._lib import Shape, Tensor
    t = Tensor(); s = Shape(); s.ndims = 2; s.dims[0] = 4; s.dims[1] = 8
    assert L.tensorfuse_allocate_tensor(byref(t), byref(s), 1, torch.cuda.current_device()) == 0
    assert t.data and t.size_bytes == 64 and t.is_contiguous
    # 2-D tensors: the operator takes [batch, seq, hidden] (tests/test_attention_gpu.py covers the computation)
    assert L.tensorfuse_fused_multi_head_attention(byref(t), byref(t), byref(t), byref(t), 4, 0.0, None) == 11
    assert L.tensorfuse_fused_multi_head_attention(byref(t), byref(t), byref(t), byref(t), 0, 0.0, None) == 1
    assert L.tensorfuse_free_tensor(byref(t)) == 0 and not t.data
    assert L.tensorfuse_free_tensor(byref(t)) == 1
    # the C++ symbols the reference's tests resolve with dlsym
    fn = getattr(L, "_ZN10tensorfuse7kernels25fused_gemm_bias_gelu_fp32EPKvS2_S2_PviiiffP11CUstream_st")
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 4 + [C.c_int] * 3 + [C.c_float] * 2 + [C.c_void_p]
    a = torch.full((8, 32), 0.1, device="cuda"); b = torch.full((32, 16), 0.1, device="cuda")
    bias = torch.full((16,), 0.1, device="cuda"); c = torch.zeros((8, 16), device="cuda")
    assert fn(a.data_ptr(), b.data_ptr(), bias.data_ptr(), c.data_ptr(), 8, 16, 32, 1.0, 1.0, None) == 0
    torch.cuda.synchronize()
    assert torch.isfinite(c).all() and float(c.abs().max()) < 10    # reference test_working_kernel.cu:124-135


def test_python_api_paths(tf, oracle):
    from tensorfuse_b200 import workloads
    x, w, b = workloads.gemm_fp32_quickstart(batch=2, seq=16, hidden=96, ffn=160)
    want = oracle.gemm_bias_gelu_f32(x.reshape(-1, 96), w, b).reshape(2, 16, 160)
    out = tf.fused_gemm_bias_gelu(x, w, b)                      # numpy, 3-D quick-start form
    np.testing.assert_allclose(out, want, rtol=1e-4, atol=1e-4)
    tx, tw, tb = (torch.from_numpy(v).cuda() for v in (x, w, b))
    tout = tf.fused_gemm_bias_gelu(tx, tw, tb)                  # CUDA tensors, in place
    torch.cuda.synchronize()
    assert np.array_equal(tout.cpu().numpy(), out)
    cpu_out = tf.fused_gemm_bias_gelu(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(b))
    assert np.array_equal(cpu_out.numpy(), out)
    # INT8 through python: explicit scales, FP16 output
    A, W, bias, sa, sw = workloads.gemm_int8(M=256, K=256, N=512)
    o16 = tf.fused_gemm_bias_gelu(A, W, bias, scales=(sa, sw), out_dtype=np.float16)
    want16 = oracle.i8_epilogue_f16(oracle.gemm_i8_acc(A, W), bias, sa, sw)
    assert oracle.f16_parity_violations(o16, want16) == 0
    with pytest.raises(RuntimeError, match="Invalid tensor shape"):
        tf.fused_gemm_bias_gelu(x, w[:, :8], b)


def test_cuda_tensor_results_are_validated_before_their_pointers_are_used(tf):
    """Caller-supplied CUDA result tensors reach the library as raw pointers: a
    wrong shape, type, layout or device must be refused in Python, not written through."""
    x = torch.randn(2, 3, 8, 64, device="cuda", dtype=torch.float16)
    good_out, good_mask = torch.empty_like(x), torch.empty(x.shape, dtype=torch.uint8, device="cuda")
    bad = [(torch.empty(2, 3, 8, 32, device="cuda", dtype=torch.float16), good_mask),      # short rows
           (torch.empty(x.shape, device="cuda", dtype=torch.float32), good_mask),          # wrong type
           (torch.empty(2, 3, 64, 8, device="cuda", dtype=torch.float16).transpose(2, 3), good_mask),  # strided
           (good_out, torch.empty(x.shape, dtype=torch.int32, device="cuda")),             # 4-byte mask
           (good_out, torch.empty(x.shape, dtype=torch.uint8)),                            # host mask
           (good_out, torch.empty(2, 3, 8, 16, dtype=torch.uint8, device="cuda"))]         # small mask
    for seed in (None, 7):
        for out, mask in bad:
            with pytest.raises(RuntimeError, match="Invalid tensor shape"):
                tf.fused_softmax_dropout(x, out, mask, 0.1, seed=seed)
            with pytest.raises(RuntimeError, match="Invalid tensor shape"):
                tf.fused_softmax_dropout_masked(x, 1.0, None, 0.1, out, mask, seed=seed)
    o, m = tf.fused_softmax_dropout(x, good_out, good_mask, 0.0, seed=7)
    torch.cuda.synchronize()
    assert o is good_out and m is good_mask and bool((m == 1).all())
    a = torch.randn(4, 16, 64, device="cuda", dtype=torch.float16)
    w = torch.randn(64, 128, device="cuda", dtype=torch.float16)
    b = torch.zeros(128, device="cuda", dtype=torch.float16)
    for out in (torch.empty(4, 16, 64, device="cuda", dtype=torch.float16),
                torch.empty(4, 128, 16, device="cuda", dtype=torch.float16).transpose(1, 2),
                torch.empty(4, 16, 128, dtype=torch.float16)):
        with pytest.raises(RuntimeError, match="Invalid tensor shape"):
            tf.fused_gemm_bias_gelu(a, w, b, out)
    with pytest.raises(RuntimeError, match="Invalid tensor shape"):
        tf.fused_gemm_bias_gelu(a, w[:32], b)
    q8 = torch.randint(-5, 5, (32, 64), device="cuda", dtype=torch.int8)
    w8 = torch.randint(-5, 5, (64, 128), device="cuda", dtype=torch.int8)
    with pytest.raises(RuntimeError, match="Invalid tensor shape"):
        tf.fused_gemm_bias_gelu(q8, w8, b.float(), torch.empty(32, 64, device="cuda", dtype=torch.float16),
                                scales=(0.1, 0.1))
    with pytest.raises(RuntimeError, match="Invalid tensor shape"):
        tf.add_layernorm(a, None, torch.ones(64, device="cuda", dtype=torch.float16),
                         torch.zeros(64, device="cuda", dtype=torch.float16), output=torch.empty(4, 16, 32, device="cuda",
                                                                                                  dtype=torch.float16))


def test_config1_full_size_through_the_struct_entry(tf, oracle):
    """Benchmark configuration 1 exactly: X[32,128,768] ~ N(0,1), W[768,3072] ~ N(0,1/768),
    b ~ N(0, 0.02^2), seed 0, FP32, 3-D tensors through tensorfuse_fused_gemm_bias_gelu; the
    whole output against the CPU loop at the reference's tolerance
    (reference src/tests/test_kernels.cu:139: max abs error < 1e-4)."""
    from gpu_util import L, byref, c_tensor, check_watchdog, dev, host, stream
    from tensorfuse_b200 import workloads
    x, w, b = workloads.gemm_fp32_quickstart()
    assert x.shape == (32, 128, 768) and w.shape == (768, 3072) and b.shape == (3072,)
    dx, dw, db = dev(x), dev(w), dev(b)
    out = torch.full((32, 128, 3072), float("nan"), dtype=torch.float32, device="cuda")
    ti, tw, tb, to = c_tensor(dx), c_tensor(dw), c_tensor(db), c_tensor(out)
    assert L.tensorfuse_fused_gemm_bias_gelu(byref(ti), byref(tw), byref(tb), byref(to), stream()) == 0
    check_watchdog()
    got = host(out).reshape(-1, 3072)
    want = oracle.gemm_bias_gelu_f32(x.reshape(-1, 768), w, b)
    assert np.isfinite(got).all()
    assert float(np.max(np.abs(got - want))) < 1e-4

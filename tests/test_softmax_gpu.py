"""fused_softmax_dropout on the GPU against the CPU oracle.

Parity bar: bit-exact.  The kernel's arithmetic (polynomial exponential,
summation schedule, IEEE reciprocal, Philox stream) is reproduced operation by
operation by oracle.softmax_dropout_exact, so outputs and masks are compared
with array_equal; the reference's own looser checks (1e-4 against numpy, row
sums, keep rate within 0.05) are asserted as well.
"""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _sched(tf, L, dtype, aligned=True):
    return tf.softmax_schedule(L, dtype, aligned)


def _exact(oracle, tf, x, p=0.0, seed=0, first_row=0, aligned=True):
    vec, warps = _sched(tf, x.shape[-1], x.dtype, aligned)
    return oracle.softmax_dropout_exact(x, p=p, seed=seed, first_row=first_row, vec=vec, warps=warps)


SHAPES = [
    (2, 8, 64, 64),      # the reference's test shape
    (1, 2, 16, 8),       # shortest vector row
    (2, 2, 32, 256),     # 1 unit per lane
    (2, 4, 64, 512),     # the attention shape's row length
    (1, 2, 24, 1024),
    (1, 1, 17, 2048),    # longest register-resident row
    (1, 1, 9, 4096),     # CTA-per-row, vector path
    (1, 1, 5, 8200),     # CTA-per-row, several steps per thread
    (1, 3, 7, 100),      # not a multiple of 8 -> scalar path, one warp
    (1, 1, 6, 1500),     # scalar path, eight warps
    (1, 1, 3, 1),        # single element rows
]


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("shape", SHAPES)
def test_p0_bit_exact(tf, oracle, shape, dtype):
    from gpu_util import softmax_rows
    r = np.random.default_rng(hash(shape) % 1000)
    x = r.uniform(-2, 2, shape).astype(dtype)
    st, out, mask = softmax_rows(x, p=0.0)
    assert st == 0
    want, wmask = _exact(oracle, tf, x)
    assert np.array_equal(mask, wmask) and mask.min() == 1
    assert np.array_equal(out.view(np.uint16 if dtype == np.float16 else np.uint32),
                          want.view(np.uint16 if dtype == np.float16 else np.uint32))
    # reference criteria: non-negative, rows sum to 1, close to the numpy oracle
    assert out.min() >= 0
    tol = 1e-4 if dtype == np.float32 else 2e-3
    np.testing.assert_allclose(out.astype(np.float64).sum(-1), 1.0, atol=50 * tol if dtype == np.float16 else 1e-4)
    np.testing.assert_allclose(out.astype(np.float64), oracle.np_softmax(x.astype(np.float64)), rtol=tol, atol=tol)


def test_reference_fixture(tf, oracle, golden):
    from gpu_util import softmax_rows
    x = golden["softmax_in"]
    st, out, mask = softmax_rows(x)
    assert st == 0 and mask.min() == 1
    np.testing.assert_allclose(out, golden["softmax_out"], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(out.sum(-1), 1.0, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("shape,p", [((2, 8, 64, 64), 0.1), ((2, 4, 64, 512), 0.1), ((1, 2, 8, 4096), 0.25),
                                     ((1, 3, 7, 100), 0.5), ((1, 1, 6, 1500), 0.1)])
def test_dropout_bit_exact_and_statistics(tf, oracle, shape, p, dtype):
    from gpu_util import softmax_rows
    r = np.random.default_rng(11)
    x = r.uniform(-2, 2, shape).astype(dtype)
    seed = 0x1234_5678_9ABC_DEF0
    st, out, mask = softmax_rows(x, p=p, seed=seed)
    assert st == 0
    want, wmask = _exact(oracle, tf, x, p=p, seed=seed)
    assert np.array_equal(mask, wmask)
    assert np.array_equal(out.view(np.uint8), want.view(np.uint8))
    assert set(np.unique(mask)) <= {0, 1}
    assert np.all(out[mask == 0] == 0) and out.min() >= 0
    n = mask.size
    assert abs(mask.mean() - (1 - p)) < max(0.05 if n < 20000 else 0.0, 5 * math.sqrt(p * (1 - p) / n) + 2e-5)
    # kept values are softmax * 1/(1-p)
    st0, base, _ = softmax_rows(x, p=0.0)
    kept = mask == 1
    np.testing.assert_allclose(out[kept].astype(np.float64), base[kept].astype(np.float64) / (1 - p),
                               rtol=2e-3 if dtype == np.float16 else 1e-6, atol=1e-7)
    # same seed -> same result; different seed -> different mask
    _, out2, mask2 = softmax_rows(x, p=p, seed=seed)
    assert np.array_equal(out2.view(np.uint8), out.view(np.uint8)) and np.array_equal(mask2, mask)
    _, _, mask3 = softmax_rows(x, p=p, seed=seed + 1)
    assert not np.array_equal(mask3, mask)


def test_p_one_and_invalid_p(tf):
    from gpu_util import softmax_rows
    x = np.random.default_rng(0).standard_normal((1, 1, 4, 64)).astype(np.float16)
    st, out, mask = softmax_rows(x, p=1.0, seed=3)
    assert st == 0 and mask.max() == 0 and np.all(out == 0)
    assert softmax_rows(x, p=1.5)[0] == 1 and softmax_rows(x, p=-0.1)[0] == 1


def test_masked_keys_and_fully_masked_rows(tf, oracle):
    from gpu_util import softmax_rows
    x = np.random.default_rng(5).standard_normal((2, 2, 8, 512)).astype(np.float16)
    x[0, :, :, 400:] = -np.inf       # key padding
    x[1, 0, 3, :] = -np.inf          # a fully masked row: defined as zeros
    st, out, mask = softmax_rows(x)
    want, _ = _exact(oracle, tf, x)
    assert st == 0 and np.array_equal(out.view(np.uint16), want.view(np.uint16))
    assert np.all(out[0, :, :, 400:] == 0) and np.all(out[1, 0, 3] == 0) and not np.isnan(out).any()


def test_shards_reproduce_the_whole(tf):
    """Rows are independent and the Philox counter is the global element index:
    any split of the rows gives the same bytes as one launch."""
    from gpu_util import softmax_rows
    x = np.random.default_rng(8).standard_normal((4, 2, 16, 512)).astype(np.float16)
    flat = x.reshape(-1, 512)
    _, whole, wmask = softmax_rows(flat, p=0.1, seed=77)
    begins, counts = tf.plan_shards(flat.shape[0], 3, 16)
    for b, c in zip(begins, counts):
        _, part, pmask = softmax_rows(flat[b:b + c], p=0.1, seed=77, first_row=b)
        assert np.array_equal(part.view(np.uint16), whole[b:b + c].view(np.uint16))
        assert np.array_equal(pmask, wmask[b:b + c])


def test_unaligned_pointers_take_the_scalar_path(tf, oracle):
    import torch
    from gpu_util import L, stream, host
    rows, Lr = 6, 64
    x = np.random.default_rng(2).standard_normal((rows, Lr)).astype(np.float16)
    buf = torch.zeros(rows * Lr + 8, dtype=torch.float16, device="cuda")
    view = buf[1:1 + rows * Lr]                      # 2-byte offset: not 16-byte aligned
    view.copy_(torch.from_numpy(x).cuda().flatten())
    out = torch.empty(rows * Lr, dtype=torch.float16, device="cuda")
    mask = torch.empty(rows * Lr, dtype=torch.uint8, device="cuda")
    st = L.tensorfuse_b200_softmax_dropout_rows(view.data_ptr(), out.data_ptr(), mask.data_ptr(), rows, Lr,
                                                1, 0.0, 0, 0, stream())
    torch.cuda.synchronize()
    assert st == 0
    want, _ = _exact(oracle, tf, x, aligned=False)
    assert np.array_equal(host(out).reshape(rows, Lr).view(np.uint16), want.view(np.uint16))


def test_struct_api_flat_wrapper_and_python(tf, oracle):
    import torch
    from gpu_util import L, byref, c_tensor, dev, host, stream
    x = np.random.default_rng(4).uniform(-2, 2, (2, 4, 32, 128)).astype(np.float32)
    dx = dev(x); dout = torch.empty_like(dx); dmask = torch.empty(x.shape, dtype=torch.uint8, device="cuda")
    ti, to = c_tensor(dx), c_tensor(dout)
    tf.set_random_seed(2024)
    assert L.tensorfuse_fused_softmax_dropout(byref(ti), byref(to), dmask.data_ptr(), 0.2, stream()) == 0
    torch.cuda.synchronize()
    seed = L.tensorfuse_b200_last_softmax_seed()
    want, wmask = _exact(oracle, tf, x, p=0.2, seed=seed)
    assert np.array_equal(host(dout).view(np.uint32), want.view(np.uint32)) and np.array_equal(host(dmask), wmask)
    # same seed source state -> same sequence of seeds
    tf.set_random_seed(2024)
    assert L.tensorfuse_fused_softmax_dropout(byref(ti), byref(to), dmask.data_ptr(), 0.2, stream()) == 0
    assert L.tensorfuse_b200_last_softmax_seed() == seed
    # flat wrapper: argument order (batch, seq_len, head_dim, num_heads), head_dim = softmax axis
    assert L.fused_softmax_dropout_fp32_wrapper(dx.data_ptr(), dout.data_ptr(), dmask.data_ptr(), 2, 32, 128, 4,
                                                0.2, seed, stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(dout).view(np.uint32), want.view(np.uint32))
    # validation codes of the struct API (reference src/tensorfuse_c_api.cpp:225-262)
    assert L.tensorfuse_fused_softmax_dropout(None, byref(to), dmask.data_ptr(), 0.0, None) == 1
    assert L.tensorfuse_fused_softmax_dropout(byref(ti), byref(to), dmask.data_ptr(), 1.5, None) == 1
    assert L.tensorfuse_fused_softmax_dropout(byref(ti), byref(to), None, 0.0, None) == 1
    t3 = c_tensor(dx, shape=(8, 32, 128))
    assert L.tensorfuse_fused_softmax_dropout(byref(t3), byref(to), dmask.data_ptr(), 0.0, None) == 11
    th = c_tensor(dev(x.astype(np.float16)))
    assert L.tensorfuse_fused_softmax_dropout(byref(th), byref(to), dmask.data_ptr(), 0.0, None) == 1
    # python: torch CUDA tensors in place, numpy through the host-buffer operator
    o_t, m_t = tf.fused_softmax_dropout(dx, dropout_prob=0.2, seed=seed)
    assert np.array_equal(host(o_t).view(np.uint32), want.view(np.uint32)) and np.array_equal(host(m_t), wmask)
    o_n, m_n = tf.fused_softmax_dropout(x, dropout_prob=0.2, seed=seed)
    assert np.array_equal(o_n.view(np.uint32), want.view(np.uint32)) and np.array_equal(m_n, wmask)


def test_full_attention_shape_properties(tf, oracle):
    """Config 4 at full size (32x16x512x512 FP16): size-independent properties on
    the whole tensor, bit-exact comparison on a sample of rows."""
    import torch
    from gpu_util import L, stream
    from tensorfuse_b200 import workloads
    x = workloads.attention_scores(seed=3, masked=True)
    dx = torch.from_numpy(x).cuda()
    out = torch.empty_like(dx); mask = torch.empty(x.shape, dtype=torch.uint8, device="cuda")
    rows = x.size // 512
    assert L.tensorfuse_b200_softmax_dropout_rows(dx.data_ptr(), out.data_ptr(), mask.data_ptr(), rows, 512, 1,
                                                  0.0, 3, 0, stream()) == 0
    torch.cuda.synchronize()
    assert int(mask.min()) == 1
    sums = out.float().sum(-1)
    assert float((sums - 1).abs().max()) < 2e-2 and float(out.min()) >= 0
    assert float(out[:, :, :, 384:][torch.isinf(dx[:, :, :, 384:])].abs().max()) == 0
    idx = np.random.default_rng(0).choice(rows, 2048, replace=False)
    flat_in = x.reshape(rows, 512); flat_out = out.reshape(rows, 512)
    want, _ = _exact(oracle, tf, flat_in[idx])
    assert np.array_equal(flat_out[torch.from_numpy(idx).cuda()].cpu().numpy().view(np.uint16), want.view(np.uint16))
    # p = 0.1: keep rate, zeros where dropped, idempotent for a fixed seed, split == whole
    out2 = torch.empty_like(dx); mask2 = torch.empty_like(mask)
    for o, m in ((out, mask), (out2, mask2)):
        assert L.tensorfuse_b200_softmax_dropout_rows(dx.data_ptr(), o.data_ptr(), m.data_ptr(), rows, 512, 1,
                                                      0.1, 3, 0, stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, out2) and torch.equal(mask, mask2)
    assert abs(float(mask.float().mean()) - 0.9) < 2e-4
    assert float(out[mask == 0].abs().max()) == 0
    half = rows // 2
    o3 = torch.empty_like(dx); m3 = torch.empty_like(mask)
    for b, c in ((0, half), (half, rows - half)):
        off = b * 512
        assert L.tensorfuse_b200_softmax_dropout_rows(dx.data_ptr() + 2 * off, o3.data_ptr() + 2 * off,
                                                      m3.data_ptr() + off, c, 512, 1, 0.1, 3, b, stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(o3, out) and torch.equal(m3, mask)
    want, wmask = _exact(oracle, tf, flat_in[idx[:64]], p=0.0)
    del want, wmask

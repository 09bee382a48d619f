"""tensorfuse_b200_softmax_dropout_masked: softmax(scale * x) with key-length
masking inside the kernel.  Bit-exact against the oracle's restatement (same
summation schedule, same exponential, same Philox stream)."""
import numpy as np
import pytest
import torch

from gpu_util import DT, L, check_watchdog, dev, host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,dtype", [((4, 3, 20, 512), np.float16), ((3, 2, 7, 264), np.float16),
                                         ((2, 2, 5, 4096), np.float16), ((3, 1, 9, 100), np.float16),
                                         ((4, 2, 6, 512), np.float32), ((2, 1, 3, 77), np.float32)])
@pytest.mark.parametrize("p", [0.0, 0.1])
def test_masked_softmax_is_bit_exact(tf, oracle, shape, dtype, p):
    rng = np.random.default_rng(13)
    x = (rng.standard_normal(shape) * 4).astype(dtype)
    Lr = shape[-1]
    lens = np.array([Lr, 0, Lr // 2 + 3, 1][:shape[0]], np.int32)
    out, mask = tf.fused_softmax_dropout_masked(dev(x), scale=0.125, kv_lengths=lens, dropout_prob=p, seed=17)
    check_watchdog()
    vec, warps = tf.softmax_schedule(Lr, dtype)
    want, wmask = oracle.softmax_dropout_masked_exact(x, scale=0.125, lengths=lens, p=p, seed=17, vec=vec, warps=warps)
    bits = np.uint16 if dtype == np.float16 else np.uint32
    assert np.array_equal(host(out).view(bits), want.view(bits))
    assert np.array_equal(host(mask), wmask)
    o = host(out).astype(np.float32)
    assert (o[1] == 0).all()                                   # no valid key -> zeros
    if shape[0] > 2:
        assert (o[2][..., Lr // 2 + 3:] == 0).all()            # masked tail
    if p == 0:
        assert np.abs(o[0].sum(-1) - 1).max() < 2e-3
        if shape[0] > 2:
            assert np.abs(o[2].sum(-1) - 1).max() < 2e-3


def test_masked_softmax_equals_materialised_minus_inf(tf):
    """Same result as adding -inf to pre-scaled FP32 scores and calling the plain operator."""
    rng = np.random.default_rng(14)
    x = rng.standard_normal((3, 4, 16, 256)).astype(np.float32)
    lens = np.array([256, 100, 31], np.int32)
    got, _ = tf.fused_softmax_dropout_masked(dev(x), scale=0.5, kv_lengths=lens, dropout_prob=0.2, seed=5)
    xs = x * np.float32(0.5)
    for b, n in enumerate(lens):
        xs[b, :, :, n:] = -np.inf
    want, _ = tf.fused_softmax_dropout(dev(xs), dropout_prob=0.2, seed=5)
    assert torch.equal(got, want)


def test_masked_softmax_validation(tf):
    x = torch.zeros((2, 1, 4, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="Invalid argument"):
        tf.fused_softmax_dropout_masked(x, scale=0.0)
    with pytest.raises(RuntimeError, match="Invalid tensor shape"):
        tf.fused_softmax_dropout_masked(x, kv_lengths=[1, 2, 3])

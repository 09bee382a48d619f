"""tensorfuse_fused_transformer_layer and tensorfuse_b200_add_layernorm against
the oracle's composition (the reference's entry point computes nothing:
src/tensorfuse_c_api.cpp:313-329, so parity is with the restated definition).

Tolerances: layer-normalised outputs have unit scale; the FP16 layer stores six
intermediate tensors in FP16, bound 3e-2 absolute; FP32 layer 2e-4; the
stand-alone LayerNorm 2e-3 (FP16 output rounding) / 1e-5 (FP32)."""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import DT, L, check_watchdog, dev, host, stream

pytestmark = pytest.mark.gpu


def layer_weights(H, F, dtype, seed=0, scale=3.0):
    rng = np.random.default_rng(seed)
    g = lambda *s: (rng.standard_normal(s) * 0.02 * scale).astype(dtype)
    w = {"query_weight": g(H, H), "key_weight": g(H, H), "value_weight": g(H, H), "output_weight": g(H, H),
         "query_bias": g(H), "key_bias": g(H), "value_bias": g(H), "output_bias": g(H),
         "ffn_weight1": g(H, F), "ffn_weight2": g(F, H), "ffn_bias1": g(F), "ffn_bias2": g(H),
         "ln1_weight": (1 + 0.1 * rng.standard_normal(H)).astype(dtype), "ln1_bias": g(H),
         "ln2_weight": (1 + 0.1 * rng.standard_normal(H)).astype(dtype), "ln2_bias": g(H)}
    return w


@pytest.mark.parametrize("rows,H,dtype", [(300, 1024, np.float16), (17, 256, np.float16), (64, 2048, np.float32),
                                          (9, 100, np.float16), (5, 4096, np.float32), (3, 7, np.float32)])
def test_add_layernorm(tf, oracle, rows, H, dtype):
    rng = np.random.default_rng(3)
    x, r = (rng.standard_normal((rows, H)) * 2).astype(dtype), rng.standard_normal((rows, H)).astype(dtype)
    g, b = (1 + 0.2 * rng.standard_normal(H)).astype(dtype), rng.standard_normal(H).astype(dtype)
    tol = 4e-3 if dtype == np.float16 else 1e-5
    out = host(tf.add_layernorm(dev(x), dev(r), dev(g), dev(b), eps=1e-5))
    assert np.abs(out - oracle.add_layernorm(x, r, g, b, 1e-5)).max() < tol * (1 + np.abs(b).max())
    out = host(tf.add_layernorm(dev(x), None, dev(g), dev(b), eps=1e-5))
    assert np.abs(out - oracle.add_layernorm(x, None, g, b, 1e-5)).max() < tol * (1 + np.abs(b).max())


@pytest.mark.parametrize("B,S,H,heads,F,dtype,tol", [(3, 128, 256, 4, 1024, np.float16, 3e-2),
                                                     (2, 200, 128, 2, 256, np.float16, 3e-2),
                                                     (2, 40, 64, 2, 128, np.float32, 2e-4)])
def test_layer_matches_oracle(tf, oracle, B, S, H, heads, F, dtype, tol):
    w = layer_weights(H, F, dtype)
    x = np.random.default_rng(1).standard_normal((B, S, H)).astype(dtype)
    dw = {k: dev(v) for k, v in w.items()}
    out = host(tf.fused_transformer_layer(dev(x), dw, heads, 0.0, 1e-5))
    check_watchdog()
    want = oracle.transformer_layer(x, w, heads, eps=1e-5)
    assert np.isfinite(out).all()
    assert np.abs(out - want).max() < tol
    # no activation, no biases
    out = host(tf.fused_transformer_layer(dev(x), dw, heads, 0.0, 1e-5, activation="none", use_bias=False))
    w0 = {k: (None if "_bias" in k and not k.startswith("ln") else v) for k, v in w.items()}
    want = oracle.transformer_layer(x, w0, heads, eps=1e-5, activation="none")
    assert np.abs(out - want).max() < tol
    check_watchdog()


def test_layer_dropout_uses_the_library_seed_source(tf, oracle):
    B, S, H, heads, F = 2, 128, 256, 4, 512
    w = layer_weights(H, F, np.float16, seed=2)
    x = np.random.default_rng(4).standard_normal((B, S, H)).astype(np.float16)
    dw = {k: dev(v) for k, v in w.items()}
    tf.set_random_seed(99)
    out = host(tf.fused_transformer_layer(dev(x), dw, heads, 0.25, 1e-5))
    # the same seed source, restarted, hands the same seed to the softmax+dropout entry point
    tf.set_random_seed(99)
    z = torch.zeros((1, 1, 1, 8), dtype=torch.float16, device="cuda")
    tf.fused_softmax_dropout(z, dropout_prob=0.25)
    seed = L.tensorfuse_b200_last_softmax_seed()
    want = oracle.transformer_layer(x, w, heads, p=0.25, seed=seed, eps=1e-5)
    assert np.abs(out - want).max() < 3e-2
    check_watchdog()


def test_layer_with_registered_projection_weights(tf):
    """Registering the query/key/value weights lets the layer build its fused
    [hidden, 3 x hidden] projection weight once.  The result must be bit-identical
    to the unregistered call; after the weights change, the stale fused copy is
    used until invalidate_weights is called (the contract of registration), and
    the fresh one afterwards."""
    B, S, H, heads, F = 2, 128, 256, 4, 512
    w = layer_weights(H, F, np.float16, seed=5)
    x = dev(np.random.default_rng(6).standard_normal((B, S, H)).astype(np.float16))
    dw = {k: dev(v) for k, v in w.items()}
    plain = host(tf.fused_transformer_layer(x, dw, heads, 0.0, 1e-5))
    tf.register_weights(dw["query_weight"], dw["key_weight"], dw["value_weight"])
    try:
        first = host(tf.fused_transformer_layer(x, dw, heads, 0.0, 1e-5))      # builds the fused weight
        again = host(tf.fused_transformer_layer(x, dw, heads, 0.0, 1e-5))      # reuses it
        assert np.array_equal(first, plain) and np.array_equal(again, plain)
        original = dw["query_weight"].clone()
        dw["query_weight"].mul_(0.5)                                           # weights change behind the cache
        torch.cuda.synchronize()
        stale = host(tf.fused_transformer_layer(x, dw, heads, 0.0, 1e-5))
        assert np.array_equal(stale, plain)
    finally:
        tf.invalidate_weights()
    fresh = host(tf.fused_transformer_layer(x, dw, heads, 0.0, 1e-5))
    assert not np.array_equal(fresh, plain)
    dw["query_weight"].copy_(original)
    torch.cuda.synchronize()
    assert np.array_equal(host(tf.fused_transformer_layer(x, dw, heads, 0.0, 1e-5)), plain)
    check_watchdog()


def test_layer_validation(tf):
    import tensorfuse_b200 as t
    H, F = 64, 128
    dw = {k: dev(v) for k, v in layer_weights(H, F, np.float16).items()}
    x = torch.zeros((2, 16, H), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="Invalid tensor shape"):
        tf.fused_transformer_layer(x, dw, 5, 0.0)                       # heads do not divide hidden
    with pytest.raises(RuntimeError, match="Invalid argument"):
        tf.fused_transformer_layer(x, dw, 0, 0.0)
    with pytest.raises(RuntimeError, match="Unsupported"):
        tf.fused_transformer_layer(x, dw, 2, 0.0, activation="relu")
    bad = dict(dw); bad["ffn_weight2"] = dw["ffn_weight1"]
    with pytest.raises(RuntimeError, match="Invalid tensor shape"):
        tf.fused_transformer_layer(x, bad, 2, 0.0)
    assert L.tensorfuse_fused_transformer_layer(None, None, None, None) == t.Status.INVALID_ARGUMENT

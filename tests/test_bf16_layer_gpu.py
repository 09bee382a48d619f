"""BF16 tensors through the attention kernel, the residual + LayerNorm kernel
and the whole transformer layer (the reference enumerates the type,
src/tensorfuse/types.h:52, and computes nothing with it).  BF16 keeps 8
significand bits, so the bounds are wider than the FP16 ones: attention
2e-2 + 2e-2 |want| (probabilities and output each rounded to BF16), LayerNorm
2e-2, layer 1.5e-1 on unit-scale outputs (six BF16 intermediates)."""
import numpy as np
import pytest
import torch

from gpu_util import check_watchdog

pytestmark = pytest.mark.gpu


def bf(x):
    return torch.from_numpy(np.ascontiguousarray(x, np.float32)).cuda().to(torch.bfloat16)


@pytest.mark.parametrize("B,Sq,Skv,H,hd,p", [(2, 256, 256, 4, 64, 0.0), (2, 200, 328, 2, 64, 0.2), (1, 40, 50, 2, 32, 0.0)])
def test_bf16_attention(tf, oracle, B, Sq, Skv, H, hd, p):
    rng = np.random.default_rng(31)
    q, k, v = (oracle.bf16_round(rng.standard_normal((B, S, H * hd)).astype(np.float32)) for S in (Sq, Skv, Skv))
    out = tf.fused_multi_head_attention(bf(q), bf(k), bf(v), None, H, p, seed=8)
    check_watchdog()
    assert out.dtype == torch.bfloat16
    want = oracle.attention(q, k, v, H, p=p, seed=8)
    got = out.float().cpu().numpy()
    assert (np.abs(got - want) <= 2e-2 + 2e-2 * np.abs(want)).all()


def test_bf16_layernorm(tf, oracle):
    rng = np.random.default_rng(32)
    x, r = (oracle.bf16_round(rng.standard_normal((300, 1024)).astype(np.float32)) for _ in range(2))
    g = oracle.bf16_round((1 + 0.1 * rng.standard_normal(1024)).astype(np.float32))
    b = oracle.bf16_round((0.1 * rng.standard_normal(1024)).astype(np.float32))
    out = tf.add_layernorm(bf(x), bf(r), bf(g), bf(b), eps=1e-5).float().cpu().numpy()
    assert np.abs(out - oracle.add_layernorm(x, r, g, b, 1e-5)).max() < 2e-2 * 4


def test_bf16_transformer_layer(tf, oracle):
    from test_transformer_layer_gpu import layer_weights
    B, S, H, heads, F = 2, 128, 256, 4, 1024
    w = {k: oracle.bf16_round(v) for k, v in layer_weights(H, F, np.float32, seed=5).items()}
    x = oracle.bf16_round(np.random.default_rng(6).standard_normal((B, S, H)).astype(np.float32))
    out = tf.fused_transformer_layer(bf(x), {k: bf(v) for k, v in w.items()}, heads, 0.0, 1e-5)
    check_watchdog()
    assert out.dtype == torch.bfloat16
    want = oracle.transformer_layer(x, w, heads, eps=1e-5)
    err = np.abs(out.float().cpu().numpy() - want)
    assert err.max() < 1.5e-1 and err.mean() < 1.5e-2

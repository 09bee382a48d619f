"""A BERT-style post-LN encoder forward that calls the two fused operators.

This is a *caller* of the hot path (the fifth benchmark configuration: BERT-large,
24 layers, hidden 1024, 16 heads of 64, FFN 4096, FP16, random weights), not a
model zoo: PyTorch does the projections, the attention matmuls and the layer
norms; libtensorfuse.so does
  * attention: fused_multi_head_attention straight on the fused QKV buffer (the
    probabilities never reach memory), or, with attention="unfused", the
    attention probabilities through fused_softmax_dropout on [b, heads, S, S]
    scores between two torch matmuls; with attention="layer" each layer is one
    call of tensorfuse_fused_transformer_layer (projections, attention, both
    layer norms and the FFN inside the library, no torch operator on the path),
  * FFN-up:   fused GEMM + bias + GELU,
  * FFN-down: fused GEMM + bias (activation NONE).
The batch dimension is the sharding dimension: each GPU (one process per GPU)
runs the same weights on its slice of the batch, no collective on the data path.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

import tensorfuse_b200 as tf
from ._lib import lib as _L


class EncoderConfig:
    def __init__(self, layers=24, hidden=1024, heads=16, ffn=4096, dropout=0.1, eps=1e-12):
        self.layers, self.hidden, self.heads, self.ffn, self.dropout, self.eps = layers, hidden, heads, ffn, dropout, eps
        assert hidden % heads == 0


def random_weights(cfg: EncoderConfig, device, seed: int = 4, dtype=torch.float16):
    """N(0, 0.02) matrices, N(0, 0.02) biases, LayerNorm gamma 1 / beta 0 -- the
    same on every rank (replicated weights)."""
    g = torch.Generator(device="cpu"); g.manual_seed(seed)
    def w(*shape):
        return (torch.randn(*shape, generator=g) * 0.02).to(device=device, dtype=dtype)
    layers = []
    for _ in range(cfg.layers):
        layers.append(dict(
            wqkv=w(cfg.hidden, 3 * cfg.hidden), bqkv=w(3 * cfg.hidden),
            wo=w(cfg.hidden, cfg.hidden), bo=w(cfg.hidden),
            w1=w(cfg.hidden, cfg.ffn), b1=w(cfg.ffn), w2=w(cfg.ffn, cfg.hidden), b2=w(cfg.hidden),
            ln1_g=torch.ones(cfg.hidden, device=device, dtype=dtype), ln1_b=torch.zeros(cfg.hidden, device=device, dtype=dtype),
            ln2_g=torch.ones(cfg.hidden, device=device, dtype=dtype), ln2_b=torch.zeros(cfg.hidden, device=device, dtype=dtype)))
    return layers


def gemm_bias_act(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, activation: str = "gelu") -> torch.Tensor:
    """[M,K] x [K,N] + bias, GELU or no activation, through tensorfuse_b200_gemm_bias_act."""
    M, K = x.shape
    N = w.shape[1]
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    act = 2 if activation == "gelu" else 0          # TENSORFUSE_ACTIVATION_GELU / _NONE
    st = _L.tensorfuse_b200_gemm_bias_act(x.data_ptr(), w.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K,
                                          int(tf.DataType.FLOAT16 if x.dtype == torch.float16 else tf.DataType.FLOAT32),
                                          act, 1.0, 1.0, int(torch.cuda.current_stream(x.device).cuda_stream))
    if st != 0:
        raise RuntimeError("tensorfuse_b200_gemm_bias_act failed: " + tf.get_error_string(st))
    return out


def layer_params(p: dict, cfg: EncoderConfig) -> dict:
    """The weights of one layer under the field names of TensorFuseTransformerParams
    (separate, contiguous Q/K/V projections), cached in the layer's dict."""
    if "_params" not in p:
        H = cfg.hidden
        p["_params"] = {
            "query_weight": p["wqkv"][:, :H].contiguous(), "key_weight": p["wqkv"][:, H:2 * H].contiguous(),
            "value_weight": p["wqkv"][:, 2 * H:].contiguous(), "output_weight": p["wo"],
            "query_bias": p["bqkv"][:H].contiguous(), "key_bias": p["bqkv"][H:2 * H].contiguous(),
            "value_bias": p["bqkv"][2 * H:].contiguous(), "output_bias": p["bo"],
            "ffn_weight1": p["w1"], "ffn_weight2": p["w2"], "ffn_bias1": p["b1"], "ffn_bias2": p["b2"],
            "ln1_weight": p["ln1_g"], "ln1_bias": p["ln1_b"], "ln2_weight": p["ln2_g"], "ln2_bias": p["ln2_b"]}
    return p["_params"]


def register_layer_weights(layers, cfg: EncoderConfig):
    """Registers the query/key/value projections of every layer as immutable, so
    that tensorfuse_fused_transformer_layer concatenates them once instead of on
    every call.  Undo with ``tf.invalidate_weights()`` before the weights change."""
    for p in layers:
        lp = layer_params(p, cfg)
        tf.register_weights(lp["query_weight"], lp["key_weight"], lp["value_weight"])


def layer_seed(seed: int, layer: int) -> int:
    return (seed * 1000003 + layer * 131) & 0xFFFFFFFFFFFF


def encoder_forward(x: torch.Tensor, layers, cfg: EncoderConfig, seed: int = 4, attn_chunk: int = 32,
                    keep_masks: list | None = None, attention: str = "fused") -> torch.Tensor:
    """x: [batch, seq, hidden] on a CUDA device.  Dropout is applied to the
    attention probabilities only (that is where the fused operators sit).  With
    attention="unfused" and ``keep_masks`` (a list) the per-layer dropout masks
    are appended to it; the fused operator drops the entries that
    fused_softmax_dropout drops on a [batch, heads, S, S] tensor with the seed
    ``layer_seed(seed, layer)``."""
    Bsz, S, H = x.shape
    nh, d = cfg.heads, H // cfg.heads
    scale = 1.0 / math.sqrt(d)
    if attention == "layer":
        # every layer is one call of tensorfuse_fused_transformer_layer: no torch operator on the path
        tf.set_random_seed(seed)
        h3 = x.contiguous()
        for p in layers:
            h3 = tf.fused_transformer_layer(h3, layer_params(p, cfg), nh, cfg.dropout, cfg.eps)
        return h3
    h = x.reshape(Bsz * S, H).contiguous()
    for li, p in enumerate(layers):
        qkv = torch.addmm(p["bqkv"], h, p["wqkv"])
        if attention == "fused":
            qkv3 = qkv.view(Bsz, S, 3, H)
            ctx2 = torch.empty((Bsz, S, H), dtype=h.dtype, device=h.device)
            tf.fused_multi_head_attention(qkv3[:, :, 0], qkv3[:, :, 1], qkv3[:, :, 2], ctx2, nh, cfg.dropout,
                                          seed=layer_seed(seed, li))
            ctx2 = ctx2.view(Bsz * S, H)
            attn = torch.addmm(p["bo"], ctx2, p["wo"])
            h = torch.nn.functional.layer_norm(h + attn, (H,), p["ln1_g"], p["ln1_b"], cfg.eps)
            up = gemm_bias_act(h, p["w1"], p["b1"], "gelu")
            down = gemm_bias_act(up, p["w2"], p["b2"], "none")
            h = torch.nn.functional.layer_norm(h + down, (H,), p["ln2_g"], p["ln2_b"], cfg.eps)
            continue
        qkv = qkv.view(Bsz, S, 3, nh, d)
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))      # [B, nh, S, d]
        ctx = torch.empty((Bsz, nh, S, d), dtype=h.dtype, device=h.device)
        layer_masks = []
        for b0 in range(0, Bsz, attn_chunk):
            b1 = min(Bsz, b0 + attn_chunk)
            scores = torch.matmul(q[b0:b1], k[b0:b1].transpose(-1, -2)) * scale    # [b, nh, S, S]
            probs, mask = tf.fused_softmax_dropout(scores.contiguous(), dropout_prob=cfg.dropout,
                                                   seed=layer_seed(seed, li) + b0)
            if keep_masks is not None:
                layer_masks.append(mask)
            ctx[b0:b1] = torch.matmul(probs, v[b0:b1])
        if keep_masks is not None:
            keep_masks.append(torch.cat(layer_masks, 0))
        ctx2 = ctx.permute(0, 2, 1, 3).reshape(Bsz * S, H)
        attn = torch.addmm(p["bo"], ctx2, p["wo"])
        h = torch.nn.functional.layer_norm(h + attn, (H,), p["ln1_g"], p["ln1_b"], cfg.eps)
        up = gemm_bias_act(h, p["w1"], p["b1"], "gelu")
        down = gemm_bias_act(up, p["w2"], p["b2"], "none")
        h = torch.nn.functional.layer_norm(h + down, (H,), p["ln2_g"], p["ln2_b"], cfg.eps)
    return h.view(Bsz, S, H)


def reference_forward(x: torch.Tensor, layers, cfg: EncoderConfig, masks=None) -> torch.Tensor:
    """The same network in plain PyTorch FP32 (tanh-form GELU); ``masks`` are the
    dropout masks the fused run produced, so that both runs drop the same entries."""
    Bsz, S, H = x.shape
    nh, d = cfg.heads, H // cfg.heads
    f = lambda t: t.float()
    h = f(x).reshape(Bsz * S, H)
    for li, p in enumerate(layers):
        qkv = (h @ f(p["wqkv"]) + f(p["bqkv"])).view(Bsz, S, 3, nh, d)
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        probs = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(d), dim=-1)
        if masks is not None:
            probs = probs * masks[li].float() / (1.0 - cfg.dropout)
        ctx = (probs @ v).permute(0, 2, 1, 3).reshape(Bsz * S, H)
        h = torch.nn.functional.layer_norm(h + ctx @ f(p["wo"]) + f(p["bo"]), (H,), f(p["ln1_g"]), f(p["ln1_b"]), cfg.eps)
        up = torch.nn.functional.gelu(h @ f(p["w1"]) + f(p["b1"]), approximate="tanh")
        h = torch.nn.functional.layer_norm(h + up @ f(p["w2"]) + f(p["b2"]), (H,), f(p["ln2_g"]), f(p["ln2_b"]), cfg.eps)
    return h.view(Bsz, S, H)

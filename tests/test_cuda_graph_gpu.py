"""The device-pointer operators are plain asynchronous launches on the caller's
stream, so a sequence of them can be captured into a CUDA graph and replayed
(warm-up first: the first call of each kernel sets function attributes and
encodes tensor maps on the host)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_operators_replay_from_a_cuda_graph(tf):
    from tensorfuse_b200 import bert_encoder as be
    torch.manual_seed(0)
    dev = torch.device("cuda")
    B, S, H, heads, F = 2, 128, 256, 4, 1024
    x = torch.randn((B, S, H), device=dev, dtype=torch.float16)
    w1 = (torch.randn((H, F), device=dev) / 16).half(); b1 = torch.zeros(F, device=dev, dtype=torch.float16)
    g = torch.ones(H, device=dev, dtype=torch.float16); bt = torch.zeros(H, device=dev, dtype=torch.float16)
    scores = torch.randn((B, heads, S, S), device=dev, dtype=torch.float16)

    def step():
        ctx = tf.fused_multi_head_attention(x, x, x, None, heads, 0.0)
        h = tf.add_layernorm(x, ctx, g, bt, eps=1e-5)
        up = be.gemm_bias_act(h.view(B * S, H), w1, b1, "gelu")
        pr, _ = tf.fused_softmax_dropout(scores, dropout_prob=0.0)
        return ctx, h, up, pr

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            want = step()                     # warm-up outside the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    want = [t.clone() for t in want]

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step()
    for t in outs:
        t.zero_()
    graph.replay()
    torch.cuda.synchronize()
    for got, ref in zip(outs, want):
        assert torch.equal(got, ref)
    # new input contents, same buffers: the replay recomputes
    x.copy_(torch.randn_like(x))
    ref2 = [t.clone() for t in step()]
    graph.replay()
    torch.cuda.synchronize()
    for got, ref in zip(outs[:3], ref2[:3]):
        assert torch.equal(got, ref)
    assert tf.watchdog_status() == 0

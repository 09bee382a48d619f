"""The encoder-forward caller of the hot path (benchmark configuration 5) on a
small network: fused softmax+dropout / FFN-up / FFN-down inside PyTorch glue
against the same network in plain PyTorch FP32.  FP16 storage between the
layers bounds the agreement; the tolerance is 3e-2 absolute on layer-normalised
activations (unit scale)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dropout", [0.0, 0.1])
def test_small_encoder_matches_fp32_reference(tf, dropout):
    from tensorfuse_b200 import bert_encoder as be
    cfg = be.EncoderConfig(layers=3, hidden=256, heads=4, ffn=1024, dropout=dropout)
    dev = torch.device("cuda")
    layers = be.random_weights(cfg, dev, seed=4)
    for p in layers:                      # larger weights than N(0, 0.02) so that every term matters
        for k in ("wqkv", "wo", "w1", "w2"):
            p[k].mul_(3.0)
    g = torch.Generator(device="cpu"); g.manual_seed(0)
    x = torch.randn((5, 128, cfg.hidden), generator=g).to(dev, torch.float16)
    masks = []
    with torch.no_grad():
        y = be.encoder_forward(x, layers, cfg, seed=7, attn_chunk=2, keep_masks=masks, attention="unfused")
        ref = be.reference_forward(x, layers, cfg, masks=masks if dropout > 0 else None)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all()
    assert len(masks) == cfg.layers and masks[0].shape == (5, 4, 128, 128)
    if dropout > 0:
        assert abs(float(masks[0].float().mean()) - (1 - dropout)) < 0.01
    else:
        assert int(masks[0].min()) == 1
    err = (y.float() - ref).abs().max().item()
    assert err < 3e-2, err


@pytest.mark.parametrize("mode", ["fused", "layer"])
@pytest.mark.parametrize("dropout", [0.0, 0.1])
def test_small_encoder_with_fused_attention(tf, dropout, mode):
    from tensorfuse_b200 import bert_encoder as be
    cfg = be.EncoderConfig(layers=3, hidden=256, heads=4, ffn=1024, dropout=dropout)
    dev = torch.device("cuda")
    layers = be.random_weights(cfg, dev, seed=4)
    for p in layers:
        for k in ("wqkv", "wo", "w1", "w2"):
            p[k].mul_(3.0)
    g = torch.Generator(device="cpu"); g.manual_seed(0)
    B, S = 5, 128
    x = torch.randn((B, S, cfg.hidden), generator=g).to(dev, torch.float16)
    with torch.no_grad():
        y = be.encoder_forward(x, layers, cfg, seed=7, attention=mode)
        # the decisions the fused operator makes are those of the softmax+dropout operator with the same seed
        masks = None
        if dropout > 0:
            zeros = torch.zeros((B, cfg.heads, S, S), dtype=torch.float16, device=dev)
            if mode == "layer":      # seeds come from the library's seed source, restarted at the same point
                tf.set_random_seed(7)
                masks = [tf.fused_softmax_dropout(zeros, dropout_prob=dropout)[1] for _ in range(cfg.layers)]
            else:
                masks = [tf.fused_softmax_dropout(zeros, dropout_prob=dropout, seed=be.layer_seed(7, li))[1]
                         for li in range(cfg.layers)]
        ref = be.reference_forward(x, layers, cfg, masks=masks)
    torch.cuda.synchronize()
    assert tf.watchdog_status() == 0
    err = (y.float() - ref).abs().max().item()
    assert err < 3e-2, err

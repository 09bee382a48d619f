"""CPU checks of the oracle pieces that have no golden vector in the reference
(the reference computes none of these operators): each restatement is pinned
against an independent formulation (numpy / torch on the CPU)."""
import numpy as np
import pytest


def test_attention_restatement_matches_numpy(oracle):
    rng = np.random.default_rng(0)
    B, S, H, hd = 2, 37, 3, 16
    q, k, v = (rng.standard_normal((B, S, H * hd)).astype(np.float32) for _ in range(3))
    split = lambda t: t.reshape(B, S, H, hd).transpose(0, 2, 1, 3)
    sc = split(q) @ split(k).transpose(0, 1, 3, 2) / np.sqrt(hd)
    pr = oracle.np_softmax(sc)
    ref = (pr @ split(v)).transpose(0, 2, 1, 3).reshape(B, S, H * hd)
    assert np.abs(oracle.attention(q, k, v, H) - ref).max() < 1e-6
    # dropout: the decisions are those of the softmax+dropout restatement on a [B, H, S, S] tensor
    p, seed = 0.3, 11
    _, mask = oracle.softmax_dropout_exact(sc.astype(np.float32), p=p, seed=seed, vec=1)
    ref = ((pr * mask / (1 - p)) @ split(v)).transpose(0, 2, 1, 3).reshape(B, S, H * hd)
    assert np.abs(oracle.attention(q, k, v, H, p=p, seed=seed) - ref).max() < 1e-6
    assert 0.6 < mask.mean() < 0.8
    # key lengths, including an item without any valid key
    out = oracle.attention(q, k, v, H, kv_lengths=np.array([5, 0], np.int32))
    ref0 = (oracle.np_softmax(sc[:1, :, :, :5]) @ split(v)[:1, :, :5]).transpose(0, 2, 1, 3).reshape(1, S, H * hd)
    assert np.abs(out[0] - ref0[0]).max() < 1e-6 and np.all(out[1] == 0)


def test_masked_softmax_restatement(oracle):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 2, 4, 64)).astype(np.float32)
    lens = np.array([64, 10, 0], np.int32)
    got, mask = oracle.softmax_dropout_masked_exact(x, scale=0.5, lengths=lens, p=0.0)
    xs = x * np.float32(0.5)
    for b, n in enumerate(lens):
        xs[b, ..., n:] = -np.inf
    want, _ = oracle.softmax_dropout_exact(xs, p=0.0)
    assert np.array_equal(got, want) and mask.min() == 1
    assert np.all(got[2] == 0) and np.abs(got[1].sum(-1) - 1).max() < 1e-6


def test_quantisation_recipes(oracle):
    from tensorfuse_b200 import workloads
    rng = np.random.default_rng(2)
    x = rng.standard_normal((64, 48)).astype(np.float32)
    q, s = oracle.quantize_sym_int8(x)
    q2, s2 = workloads.quantize_sym_int8(x)            # the generator of the INT8 benchmark configuration
    assert np.array_equal(q, q2) and np.float32(s2) == s
    assert np.abs(q.astype(np.float32) * s - x).max() <= s / 2 * (1 + 1e-6)
    qc, sc = oracle.quantize_sym_int8_columns(x)
    for n in range(x.shape[1]):
        qn, sn = oracle.quantize_sym_int8(x[:, n])
        assert np.array_equal(qc[:, n], qn) and sc[n] == sn
    qz, sz = oracle.quantize_sym_int8(np.zeros(5, np.float32))
    assert sz == 1 and not qz.any()


def test_bf16_and_fp8_helpers_match_torch(oracle):
    torch = pytest.importorskip("torch")
    x = np.random.default_rng(3).standard_normal(4096).astype(np.float32) * 100
    assert np.array_equal(oracle.bf16_round(x), torch.from_numpy(x).to(torch.bfloat16).float().numpy())
    assert np.array_equal(oracle.bf16_from_bits(oracle.bf16_bits(oracle.bf16_round(x))), oracle.bf16_round(x))
    table = oracle.fp8_e4m3_table()
    want = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.nan_to_num(table, nan=777.0), np.nan_to_num(want, nan=777.0))
    assert table[0x7E] == 448.0 and np.isnan(table[0x7F])


def test_layernorm_and_layer_restatements(oracle):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(4)
    B, S, H, heads, F = 2, 9, 16, 2, 32
    x = rng.standard_normal((B, S, H)).astype(np.float32)
    g = lambda *s: (rng.standard_normal(s) * 0.2).astype(np.float32)
    w = {"query_weight": g(H, H), "key_weight": g(H, H), "value_weight": g(H, H), "output_weight": g(H, H),
         "query_bias": g(H), "key_bias": g(H), "value_bias": g(H), "output_bias": g(H),
         "ffn_weight1": g(H, F), "ffn_weight2": g(F, H), "ffn_bias1": g(F), "ffn_bias2": g(H),
         "ln1_weight": 1 + g(H), "ln1_bias": g(H), "ln2_weight": 1 + g(H), "ln2_bias": g(H)}
    r = rng.standard_normal((B * S, H)).astype(np.float32)
    ln = torch.nn.functional.layer_norm(torch.from_numpy(x.reshape(-1, H)).double() + torch.from_numpy(r).double(), (H,),
                                        torch.from_numpy(w["ln1_weight"]).double(), torch.from_numpy(w["ln1_bias"]).double(), 1e-5)
    assert np.abs(oracle.add_layernorm(x.reshape(-1, H), r, w["ln1_weight"], w["ln1_bias"], 1e-5) - ln.numpy()).max() < 1e-12
    # whole layer against torch's own attention / layer-norm / gelu in float64
    t = {k: torch.from_numpy(v).double() for k, v in w.items()}
    xt = torch.from_numpy(x).double()
    proj = lambda a, n: a @ t[n + "_weight"] + t[n + "_bias"]
    heads_of = lambda a: a.view(B, S, heads, H // heads).transpose(1, 2)
    q, k, v = (heads_of(proj(xt, n)) for n in ("query", "key", "value"))
    ctx = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, S, H)
    h1 = torch.nn.functional.layer_norm(xt + proj(ctx, "output"), (H,), t["ln1_weight"], t["ln1_bias"], 1e-5)
    u = torch.nn.functional.gelu(h1 @ t["ffn_weight1"] + t["ffn_bias1"], approximate="tanh")
    out = torch.nn.functional.layer_norm(h1 + u @ t["ffn_weight2"] + t["ffn_bias2"], (H,), t["ln2_weight"], t["ln2_bias"], 1e-5)
    assert np.abs(oracle.transformer_layer(x, w, heads, eps=1e-5) - out.numpy()).max() < 1e-5

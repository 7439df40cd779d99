"""The plain implementation itself: properties that follow from the formulas (CPU)."""

import math

import pytest
import torch

import helpers
import plain_qwen3 as plain

F64 = torch.float64


def test_rmsnorm_formula_and_eps():
    x = torch.tensor([[3.0, 4.0]], dtype=F64)
    w = torch.tensor([2.0, 0.5], dtype=F64)
    got = plain.rmsnorm(x, w, 0.5)
    want = x / math.sqrt((9 + 16) / 2 + 0.5) * w
    assert torch.allclose(got, want, atol=0, rtol=1e-15)
    assert float(plain.rmsnorm(torch.zeros(1, 4, dtype=F64), torch.ones(4, dtype=F64), 1e-6).abs().max()) == 0.0


def test_rope_pairs_rotate_by_the_position_and_keep_the_norm():
    hd, theta = 8, 100.0
    x = torch.randn(5, 2, hd, dtype=F64, generator=torch.Generator().manual_seed(0))
    pos = torch.tensor([0, 1, 7, 100, 30000])
    y = plain.rope(x, pos, theta)
    assert torch.allclose(y[0], x[0], atol=1e-7)                                  # position 0: identity
    assert torch.allclose(y.pow(2).sum(-1), x.pow(2).sum(-1), rtol=1e-6)
    j = 1
    ang = 7 * theta ** (-2.0 * j / hd)
    a, b = x[2, 0, j], x[2, 0, j + hd // 2]
    assert abs(float(y[2, 0, j]) - float(a * math.cos(ang) - b * math.sin(ang))) < 1e-6
    assert abs(float(y[2, 0, j + hd // 2]) - float(b * math.cos(ang) + a * math.sin(ang))) < 1e-6
    # scores depend on the distance only
    q, k = torch.randn(1, 1, hd, dtype=F64), torch.randn(1, 1, hd, dtype=F64)
    s1 = (plain.rope(q, torch.tensor([10]), theta) * plain.rope(k, torch.tensor([4]), theta)).sum()
    s2 = (plain.rope(q, torch.tensor([506]), theta) * plain.rope(k, torch.tensor([500]), theta)).sum()
    assert abs(float(s1 - s2)) < 1e-5


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(1)
    T, n_q, n_kv, hd = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n, hd, dtype=F64, generator=g) for n in (n_q, n_kv, n_kv))
    out = plain.attention(q, k, v, hd ** -0.5)
    k2, v2 = k.clone(), v.clone()
    k2[6:] += 5.0; v2[6:] -= 3.0                              # the future changes nothing before it
    assert torch.equal(plain.attention(q, k2, v2, hd ** -0.5)[:6], out[:6])
    assert torch.allclose(out[0], v[0].repeat_interleave(2, 0))      # first token sees itself only; head h -> h // 2
    w = plain.attention(q, k, v, hd ** -0.5, window=3)
    assert torch.allclose(w[:3], out[:3]) and not torch.allclose(w[5], out[5])
    k3 = k.clone(); k3[:4] += 9.0                             # keys 0..3 lie outside token 8's window of 3
    assert torch.equal(plain.attention(q, k3, v, hd ** -0.5, window=3)[8], w[8])
    # a later chunk of queries against all keys gives the same rows
    assert torch.allclose(plain.attention(q[5:], k, v, hd ** -0.5), out[5:])


def test_one_key_that_stands_out_takes_all_the_weight():
    T, hd = 300, 16
    g = torch.Generator().manual_seed(2)
    q = torch.randn(1, 1, hd, dtype=F64, generator=g)
    k = torch.randn(T, 1, hd, dtype=F64, generator=g) * 0.1
    v = torch.randn(T, 1, hd, dtype=F64, generator=g)
    k[17, 0] = q[0, 0] * 40.0
    out = plain.attention(q, k, v, 1.0)
    assert torch.allclose(out[0, 0], v[17, 0], atol=1e-9)


def test_forward_is_causal_and_window_config_matters(model_dirs):
    cfg, w = plain.read_model(model_dirs("B"))
    ids = helpers.rand_ids(120, cfg["vocab_size"], 3)
    full = plain.forward(cfg, w, ids)
    assert full.shape == (120, 320)
    assert torch.allclose(plain.forward(cfg, w, ids[:50]), full[:50], atol=1e-10)
    nowin = dict(cfg, use_sliding_window=False)
    other = plain.forward(nowin, w, ids)
    assert torch.allclose(other[:80], full[:80], atol=1e-10) and not torch.allclose(other[100:], full[100:], atol=1e-6)


def test_tied_and_untied_heads(model_dirs):
    cfg, w = plain.read_model(model_dirs("A"))
    assert "lm_head.weight" not in w and cfg["tie_word_embeddings"]
    x = torch.randn(3, 64, dtype=F64)
    assert torch.equal(plain.head(x, w, cfg), plain.rmsnorm(x, w["model.norm.weight"], 1e-6) @ w["model.embed_tokens.weight"].T)
    cfgb, wb = plain.read_model(model_dirs("B"))
    assert "lm_head.weight" in wb and not torch.equal(wb["lm_head.weight"], wb["model.embed_tokens.weight"])


def test_pick_breaks_ties_low_and_sampling_is_seeded():
    lg = torch.tensor([0.0, 2.0, 2.0, 1.0])
    assert plain.pick(lg) == 1
    lg = torch.randn(50, generator=torch.Generator().manual_seed(0))
    a = [plain.pick(lg, 0.8, seed=5, request=1, step=s) for s in range(20)]
    assert a == [plain.pick(lg, 0.8, seed=5, request=1, step=s) for s in range(20)]
    assert a != [plain.pick(lg, 0.8, seed=6, request=1, step=s) for s in range(20)]
    assert len(set(a)) > 3
    # the draw follows softmax(logits / T): a dominant logit wins nearly always
    lg2 = torch.zeros(50); lg2[9] = 12.0
    assert sum(plain.pick(lg2, 1.0, 0, 0, s) == 9 for s in range(40)) >= 39


def test_schedule_with_a_layer_twice_and_a_shared_cache(model_dirs):
    cfg, w = plain.read_model(model_dirs("A"))
    ids = helpers.rand_ids(12, 256, 4)
    base = plain.forward(cfg, w, ids)
    twice = plain.forward(cfg, w, ids, schedule=[(0, 0, True), (1, 1, True), (1, 2, True)])
    shared = plain.forward(cfg, w, ids, schedule=[(0, 0, True), (1, 1, True), (1, 1, False)])
    assert not torch.allclose(base, twice) and not torch.allclose(twice, shared)

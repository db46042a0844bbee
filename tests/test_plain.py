"""The plain implementation checked against itself and against elementary identities."""
import math

import torch

import plain_qwen3 as plain
from helpers import random_tokens


def test_rms_norm_and_head_norm():
    x = torch.randn(5, 12, dtype=torch.float64)
    g = torch.rand(12, dtype=torch.float64) + 0.5
    y = plain.rms_norm(x, g, 1e-5)
    for r in range(5):
        inv = 1.0 / math.sqrt(float((x[r] ** 2).sum()) / 12 + 1e-5)
        assert torch.allclose(y[r], x[r] * inv * g, atol=1e-14)
    h = torch.randn(3, 4, 8, dtype=torch.float64)
    gh = torch.rand(8, dtype=torch.float64)
    yh = plain.head_rms_norm(h, gh, 1e-6)
    assert torch.allclose(yh[2, 1], plain.rms_norm(h[2, 1][None], gh, 1e-6)[0], atol=1e-14)


def test_rotation_pairs_halves_and_keeps_relative_position():
    d = 16
    x = torch.randn(1, 1, d, dtype=torch.float64)
    y = plain.rotary_half_split(x.repeat(4, 1, 1), [0, 1, 5, 9], 1e4)
    assert torch.allclose(y[0], x[0], atol=1e-15)                      # position 0: no rotation
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1).expand(4, 1), atol=1e-12)
    # pair (i, i + d/2) turns by p * theta^(-2i/d); element 3 pairs with 11, not with 2 or 4
    p, i = 5, 3
    a = p * 1e4 ** (-2 * i / d)
    want = x[0, 0, i] * math.cos(a) - x[0, 0, i + d // 2] * math.sin(a)
    assert abs(float(y[2, 0, i] - want)) < 1e-6
    q = torch.randn(1, 1, d, dtype=torch.float64); k = torch.randn(1, 1, d, dtype=torch.float64)
    def dot(pq, pk):
        return float((plain.rotary_half_split(q, [pq], 1e4) * plain.rotary_half_split(k, [pk], 1e4)).sum())
    assert abs(dot(7, 3) - dot(14, 10)) < 1e-5                         # depends on the distance only


def test_attention_matches_softmax_and_groups_heads():
    T, nq, nkv, d = 6, 4, 2, 8
    q = torch.randn(T, nq, d, dtype=torch.float64); k = torch.randn(T, nkv, d, dtype=torch.float64)
    v = torch.randn(T, nkv, d, dtype=torch.float64)
    out = plain.causal_attention(q, k, v, nq, nkv)
    for j in range(nq):
        g = j // 2
        s = (q[:, j] @ k[:, g].t()) / math.sqrt(d)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
        assert torch.allclose(out[:, j], torch.softmax(s, -1) @ v[:, g], atol=1e-12)
    w = plain.causal_attention(q, k, v, nq, nkv, window=2)
    s = (q[:, 0] @ k[:, 0].t()) / math.sqrt(d)
    keep = torch.tril(torch.ones(T, T, dtype=torch.bool)) & ~torch.tril(torch.ones(T, T, dtype=torch.bool), -2)
    assert torch.allclose(w[:, 0], torch.softmax(s.masked_fill(~keep, -math.inf), -1) @ v[:, 0], atol=1e-12)


def test_swiglu_and_greedy_rules():
    g = torch.tensor([-2.0, 0.0, 3.0], dtype=torch.float64); u = torch.tensor([1.5, 2.0, -1.0], dtype=torch.float64)
    assert torch.allclose(plain.swiglu(g, u), torch.nn.functional.silu(g) * u, atol=1e-15)
    assert plain.greedy(torch.tensor([1.0, 5.0, 5.0, float("nan"), float("inf")])) == 1   # lowest index, finite only
    assert plain.greedy(torch.tensor([float("nan")] * 3)) == 0
    logits = torch.tensor([0.0, 1.0, float("-inf"), 2.0])
    cdf = plain.temperature_cdf(logits, 0.5)
    assert cdf[2] == cdf[1] and abs(float(cdf[-1]) - 1.0) < 1e-12
    assert plain.temperature_sample(logits, 0.5, 0.0) == 0
    assert plain.temperature_sample(logits, 0.5, float(cdf[1]) + 1e-9) == 3
    assert plain.temperature_sample(logits, 0.5, 0.999999) == 3


def test_whole_model_is_causal_and_32_bit_agrees_with_64_bit(model_dirs):
    for name in ("A", "B"):
        cfg, w = plain.load_folder(model_dirs[(name, "float32")])
        toks = random_tokens(cfg["vocab_size"], 12, 3)
        full = plain.model_logits(cfg, w, toks)
        assert full.shape == (12, cfg["vocab_size"])
        part = plain.model_logits(cfg, w, toks[:7])
        assert torch.allclose(full[:7], part, atol=1e-12)              # later tokens change nothing earlier
        f32 = plain.model_logits(cfg, w, toks, dtype=torch.float32)
        assert (f32.double() - full).abs().max() < 2e-5 * full.abs().max()
    cfg, w = plain.load_folder(model_dirs[("A", "float32")])
    assert "lm_head.weight" not in w                                   # tied: the embedding is the head
    out, why = plain.generate_greedy(cfg, w, [1, 2, 3], 4)
    assert len(out) == 4 and why == "max_new_tokens"
    out2, why2 = plain.generate_greedy(cfg, w, [1, 2, 3], 4, stop_ids=(out[2],))
    assert out2 == out[:out.index(out[2])] and why2 == "eos"

"""The plain implementation against itself and against hand-made cases (no GPU)."""
import math

import pytest
import torch

import plain_qwen2 as P
from engine_fixtures import model_dir, plain_model


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    out = P.rms_norm(x, torch.tensor([2.0, 0.5], dtype=torch.float64), 0.0)
    s = 1 / math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[3 * s * 2, 4 * s * 0.5]], dtype=torch.float64))


def test_rope_pairs_i_with_i_plus_half_and_keeps_the_tail():
    x = torch.zeros(1, 1, 6, dtype=torch.float64)
    x[0, 0] = torch.tensor([1.0, 2.0, 3.0, 4.0, 9.0, 9.5])
    out = P.rope_neox(x, torch.tensor([3]), theta=100.0, rotary_dim=4)
    a0, a1 = 3.0, 3.0 * 100.0 ** (-0.5)
    exp = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
           1 * math.sin(a0) + 3 * math.cos(a0), 2 * math.sin(a1) + 4 * math.cos(a1), 9.0, 9.5]
    assert torch.allclose(out[0, 0], torch.tensor(exp, dtype=torch.float64))
    assert torch.equal(P.rope_neox(x, torch.tensor([0]), 100.0, 4), x)


def test_attention_mask_window_and_groups():
    T, H, Hkv, d = 6, 4, 2, 2
    g = torch.Generator().manual_seed(0)
    q = torch.randn(T, H, d, generator=g, dtype=torch.float64)
    k = torch.randn(T, Hkv, d, generator=g, dtype=torch.float64)
    v = torch.randn(T, Hkv, d, generator=g, dtype=torch.float64)
    out = P.attention(q, k, v, 0.7, None)
    assert torch.allclose(out[0, :2], v[0, 0].expand(2, d)) and torch.allclose(out[0, 2:], v[0, 1].expand(2, d))
    # by hand for the last query, head 3 (kv head 1), window 3: keys 3, 4, 5
    w = P.attention(q, k, v, 0.7, 3)
    s = torch.stack([(q[5, 3] * k[j, 1]).sum() * 0.7 for j in (3, 4, 5)])
    p = torch.softmax(s, 0)
    assert torch.allclose(w[5, 3], p[0] * v[3, 1] + p[1] * v[4, 1] + p[2] * v[5, 1])
    assert torch.allclose(w[:3], out[:3]) and not torch.allclose(w[5], out[5])


@pytest.mark.parametrize("name", ["A", "B"])
def test_logits_of_a_prefix_do_not_change_when_tokens_follow(name):
    cfg, w = plain_model(model_dir(name))
    toks = [(7 * i + 3) % cfg["vocab_size"] for i in range(70)]
    full = P.forward(cfg, w, toks)
    part = P.forward(cfg, w, toks[:25])
    assert full.shape == (70, cfg["vocab_size"])
    assert torch.allclose(full[:25], part, atol=1e-12)


def test_window_changes_late_positions_only():
    cfg, w = plain_model(model_dir("B"))
    toks = [(11 * i + 5) % 1000 for i in range(80)]
    a = P.forward(cfg, w, toks)
    b = P.forward(dict(cfg, use_sliding_window=False), w, toks)
    assert torch.allclose(a[:48], b[:48], atol=1e-12)          # window 48: positions < 48 see everything
    assert (a[60:] - b[60:]).abs().max() > 1e-9


def test_tied_head_is_the_embedding():
    cfg, w = plain_model(model_dir("A"))
    assert "lm_head.weight" not in w
    out = P.forward(cfg, w, [1, 2, 3])
    assert out.shape == (3, 512)
    g = P.greedy_generate(cfg, w, [1, 2, 3], 4)
    assert len(g) == 4 and all(0 <= t < 512 for t in g)

"""The plain implementation's own properties, after the reference's operator tests
(crates/vipera-backend-cpu/src/model.rs:4465-4538, 5451-5508, 6014-6118): the norm matches
its definition, rotation by position 0 is the identity and keeps lengths, attention is causal
and ignores later positions, query heads share the KV head of their group, a window hides
what lies before it, and the whole model's logits at a position depend only on the tokens up
to it."""
import math

import pytest
import torch

import helpers
import plain_qwen2 as plain


def test_rms_norm_definition():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=torch.float64)
    out = plain.rms_norm(x, w, 0.0)
    scale = 1.0 / math.sqrt((9 + 16) / 4)
    assert torch.allclose(out, torch.tensor([[3 * scale, 8 * scale, 0.0, 0.0]], dtype=torch.float64))
    assert torch.allclose(plain.rms_norm(x * 5, w, 0.0), out)          # scale invariance without eps


def test_rope_rotates_pairs_by_the_position_angle():
    d = 8
    sin, cos = plain.rope_angles([0, 1, 5], d, 10000.0)
    x = torch.randn(3, 2, d, dtype=torch.float64)
    out = plain.rope_neox(x, sin, cos)
    assert torch.allclose(out[0], x[0])                                  # position 0 is the identity
    assert torch.allclose(out.norm(dim=-1), x.norm(dim=-1))             # a rotation keeps lengths
    angle = 5.0 / (10000.0 ** (2.0 * 1 / d))                             # pair (1, 1 + d/2) at position 5
    a, b = x[2, 0, 1], x[2, 0, 1 + d // 2]
    assert math.isclose(float(out[2, 0, 1]), float(a * math.cos(angle) - b * math.sin(angle)), rel_tol=1e-5)
    assert math.isclose(float(out[2, 0, 1 + d // 2]), float(a * math.sin(angle) + b * math.cos(angle)), rel_tol=1e-5)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    heads, kv_heads, d, n = 4, 2, 8, 12
    q = torch.randn(n, heads, d, dtype=torch.float64)
    k = torch.randn(n, kv_heads, d, dtype=torch.float64)
    v = torch.randn(n, kv_heads, d, dtype=torch.float64)
    out = plain.attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[7:], v2[7:] = 99.0, -99.0                                         # later positions do not matter
    assert torch.allclose(plain.attention(q, k2, v2)[:7], out[:7])
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])   # one key: its value
    q_same = q.clone()
    q_same[:, 1] = q_same[:, 0]                                          # heads 0 and 1 share KV head 0
    shared = plain.attention(q_same, k, v)
    assert torch.allclose(shared[:, 0], shared[:, 1])
    windowed = plain.attention(q, k, v, window=3)
    k3, v3 = k.clone(), v.clone()
    k3[:8], v3[:8] = 50.0, 50.0                                          # out of the window of position 10
    assert torch.allclose(plain.attention(q, k3, v3, window=3)[10:], windowed[10:])
    assert not torch.allclose(windowed[10], out[10])
    tail = plain.attention(q[9:], k, v, first_position=9)               # queries may start later than keys
    assert torch.allclose(tail, out[9:])


def test_silu_and_swiglu():
    x = torch.tensor([-2.0, 0.0, 3.0], dtype=torch.float64)
    assert torch.allclose(plain.silu(x), x * torch.sigmoid(x))
    h = torch.randn(2, 4, dtype=torch.float64)
    gate, up, down = (torch.randn(6, 4, dtype=torch.float64), torch.randn(6, 4, dtype=torch.float64),
                      torch.randn(4, 6, dtype=torch.float64))
    want = ((h @ up.T) * plain.silu(h @ gate.T)) @ down.T
    assert torch.allclose(plain.swiglu(h, gate, up, down), want)


@pytest.mark.parametrize("name", ["A", "B"])
def test_logits_at_a_position_depend_only_on_the_prefix(name):
    folder = helpers.model_folder(name, "float32")
    config, weights = helpers.plain_model(folder)
    assert config["layers"] == helpers.CONFIGS[name]["num_hidden_layers"]
    tokens = helpers.random_tokens(config["vocab"], 40, 5)
    whole = plain.forward(config, weights, tokens)
    assert whole.shape == (40, config["vocab"]) and torch.isfinite(whole).all()
    prefix = plain.forward(config, weights, tokens[:25])
    assert torch.allclose(whole[:25], prefix, atol=1e-10)
    changed = list(tokens)
    changed[30] = (changed[30] + 1) % config["vocab"]
    other = plain.forward(config, weights, changed)
    assert torch.allclose(other[:30], whole[:30], atol=1e-10) and not torch.allclose(other[30:], whole[30:])
    single = plain.forward(config, weights, tokens, dtype=torch.float32)
    assert float((single.double() - whole).abs().max()) < 1e-4 * float(whole.abs().max())
    greedy = plain.greedy_continuation(config, weights, tokens[:5], 3)
    assert len(greedy) == 3 and greedy[0] == int(torch.argmax(plain.forward(config, weights, tokens[:5])[-1]))


def test_tied_and_untied_output_and_windows():
    a = plain.read_config(helpers.model_folder("A", "float32"))
    b = plain.read_config(helpers.model_folder("B", "float32"))
    assert a["windows"] == [None, None] and b["windows"] == [None, 80, 80]
    assert "lm_head.weight" not in helpers.plain_model(helpers.model_folder("A", "float32"))[1]
    assert "lm_head.weight" in helpers.plain_model(helpers.model_folder("B", "float32"))[1]
    # a schedule that runs layer 0 twice and lets layer 1 read layer 0's cache is another model
    config, weights = helpers.plain_model(helpers.model_folder("A", "float32"))
    tokens = helpers.random_tokens(config["vocab"], 9, 1)
    base = plain.forward(config, weights, tokens)
    twice = plain.forward(config, weights, tokens, schedule=[(0, 0, True), (0, 1, True), (1, 0, False)])
    assert twice.shape == base.shape and not torch.allclose(twice, base)

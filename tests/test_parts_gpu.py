"""Each part alone against the plain implementation, and the seams that let another part or
architecture in: a toy mixer with state of its own, a toy position encoding and a toy
architecture whose execution order names a layer twice and lets a layer read another's cache,
all defined here and registered without a change to the package's files."""
import json
import math
import os
import tempfile

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _pkg():
    import vipera_rs_b200
    from vipera_rs_b200 import parts  # noqa: F401

    return vipera_rs_b200


class _Host:
    """What the runner needs to know of a model to build a step's context for one part."""

    def __init__(self, dtype, vocab=1000, hidden=64, positions=4096):
        from types import SimpleNamespace

        self.dtype, self.device = dtype, torch.device(DEV)
        self.spec = SimpleNamespace(vocab_size=vocab, hidden_size=hidden, max_position_embeddings=positions)
        self.graph_safe = False


def _context(dtype, cache_requests, entries, page_size=16, pages=64, slots=4):
    """entries: [(request id, first position, count, fresh)]; pages are reserved for them."""
    _pkg()
    from vipera_rs_b200.cache import CachePools
    from vipera_rs_b200.engine import ModelRunner, StepInput

    host = _Host(dtype)
    pools = CachePools(cache_requests, page_size=page_size, num_pages=pages, num_state_slots=slots, dtype=dtype,
                       device=DEV)
    pools.poison()
    runner = ModelRunner(host, pools, max_model_len=4096)
    return pools, runner


def _step(pools, runner, entries):
    from vipera_rs_b200.engine import StepInput

    manager = pools.manager
    for request, first, count, _ in entries:
        if not manager.is_open(request):
            manager.open(request)
        manager.reserve(request, first + count)
    total = sum(count for _, _, count, _ in entries)
    step = StepInput(requests=[e[0] for e in entries], tokens=np.zeros(total, dtype=np.int32),
                     counts=[e[2] for e in entries], pos0=[e[1] for e in entries], fresh=[e[3] for e in entries],
                     logit_rows=np.zeros(0, dtype=np.int32))
    ctx = runner.build_context(step, runner.model.dtype)
    return ctx


def _commit(pools, entries):
    for request, first, count, _ in entries:
        pools.manager.commit(request, first + count)


def _rel(got, want):
    return float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max())


LIMIT = {torch.float32: 3e-6, torch.bfloat16: 2e-2}


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_and_rotary_parts(dtype):
    _pkg()
    from vipera_rs_b200.config import NORMS, POSITION_ENCODINGS

    torch.manual_seed(1)
    size, eps = 200, 3e-5
    weight = 1 + 0.1 * torch.randn(size)
    norm = NORMS.find("rmsnorm")({"size": size, "eps": eps}, "n", {"n.weight": weight}, dtype, DEV)
    x = torch.randn(9, size, device=DEV) * 2
    out = torch.empty(9, size, device=DEV, dtype=dtype)
    norm.forward(None, x, out)
    assert _rel(out, plain.rms_norm(x.cpu().double(), weight.double(), eps)) < LIMIT[dtype]
    rope = POSITION_ENCODINGS.find("rope_neox")({"head_dim": 48, "theta": 50000.0, "max_positions": 300}, "", {},
                                                dtype, DEV)
    cos, sin = rope.tables()
    want_sin, want_cos = plain.rope_angles(range(300), 48, 50000.0)
    assert torch.equal(cos.cpu(), want_cos) and torch.equal(sin.cpu(), want_sin)   # the same 32-bit angles


def _attention_tensors(hidden, heads, kv_heads, d, bias, seed):
    g = torch.Generator().manual_seed(seed)
    t = {
        "a.q_proj.weight": torch.randn(heads * d, hidden, generator=g) * 0.08,
        "a.k_proj.weight": torch.randn(kv_heads * d, hidden, generator=g) * 0.08,
        "a.v_proj.weight": torch.randn(kv_heads * d, hidden, generator=g) * 0.08,
        "a.o_proj.weight": torch.randn(hidden, heads * d, generator=g) * 0.08,
    }
    if bias:
        for name, width in (("q", heads * d), ("k", kv_heads * d), ("v", kv_heads * d)):
            t[f"a.{name}_proj.bias"] = torch.randn(width, generator=g) * 0.1
    return t


def _plain_attention_part(tensors, h, heads, kv_heads, d, theta, window, bias, round_to):
    """x -> o_proj(attention(rope(q), rope(k), v)) for one whole sequence, by the plain functions."""
    n = h.shape[0]
    rounded = lambda v: v if round_to is None else v.to(round_to).to(v.dtype)  # noqa: E731
    w = {k: rounded(v.double()) for k, v in tensors.items() if k.endswith("weight")}
    project = lambda name: h @ w[f"a.{name}_proj.weight"].T + (tensors[f"a.{name}_proj.bias"].double() if bias else 0)  # noqa: E731
    sin, cos = plain.rope_angles(range(n), d, theta)
    q = rounded(plain.rope_neox(project("q").view(n, heads, d), sin, cos))
    k = rounded(plain.rope_neox(project("k").view(n, kv_heads, d), sin, cos))
    v = rounded(project("v").view(n, kv_heads, d))
    mixed = rounded(plain.attention(q, k, v, window=window).reshape(n, heads * d))
    return mixed @ w["a.o_proj.weight"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,d,window,bias", [(4, 2, 64, None, True), (3, 1, 128, 40, True),
                                                          (5, 5, 48, None, False)])
def test_attention_part_in_portions(dtype, heads, kv_heads, d, window, bias):
    """The attention mixer alone: a sequence fed whole, and the same sequence in portions of
    17, 2 and 1 tokens beside a second request, give the plain result."""
    pkg = _pkg()
    from vipera_rs_b200.config import MIXERS, PartSpec

    hidden, theta, n = 96, 10000.0, 70
    tensors = _attention_tensors(hidden, heads, kv_heads, d, bias, seed=heads * 7 + d)
    params = {"hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": d, "qkv_bias": bias,
              "window": window, "softmax_scale": 1 / math.sqrt(d),
              "position": PartSpec("rope_neox", {"head_dim": d, "theta": theta, "max_positions": 512})}
    mixer = MIXERS.find("gqa_attention")(params, "a", tensors, dtype, DEV)
    assert mixer.cache_request() == pkg.parts.PagedKV(kv_heads, d, window)
    torch.manual_seed(3)
    round_to = torch.bfloat16 if dtype == torch.bfloat16 else None
    sequences = {0: torch.randn(n, hidden).to(dtype).double(), 1: torch.randn(33, hidden).to(dtype).double()}
    want = {r: _plain_attention_part(tensors, h, heads, kv_heads, d, theta, window, bias, round_to)
            for r, h in sequences.items()}
    pools, runner = _context(dtype, {0: mixer.cache_request()}, [])
    done = {0: 0, 1: 0}
    got = {r: torch.zeros(len(h), hidden, dtype=torch.float64) for r, h in sequences.items()}
    plan = [[(0, 17), (1, 33)], [(0, 2)], [(0, 1)], [(0, 1)], [(0, 30)], [(0, 19)]]
    for portions in plan:
        entries = [(r, done[r], count, 1 if done[r] == 0 else 0) for r, count in portions]
        ctx = _step(pools, runner, entries)
        h = torch.cat([sequences[r][first:first + count] for r, first, count, _ in entries]).to(DEV, dtype)
        residual = torch.zeros(h.shape[0], hidden, device=DEV)
        mixer.forward(ctx, h, residual, pools.views[0], True)
        torch.cuda.synchronize()
        offset = 0
        for r, first, count, _ in entries:
            got[r][first:first + count] = residual[offset:offset + count].double().cpu()
            offset += count
            done[r] += count
        _commit(pools, entries)
    for r in sequences:
        assert done[r] == len(sequences[r])
        assert _rel(got[r], want[r]) < LIMIT[dtype], f"request {r}"
    if window:
        assert pools.manager.stats(0)["used_pages"] < -(-n // 16) + -(-33 // 16)   # the window gave pages back


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens", [3, 200])
def test_feed_forward_and_block_parts(dtype, tokens):
    _pkg()
    from vipera_rs_b200.config import BLOCKS, FEED_FORWARDS, LayerSpec, PartSpec

    hidden, inter = 96, 176
    g = torch.Generator().manual_seed(tokens)
    tensors = {"m.gate_proj.weight": torch.randn(inter, hidden, generator=g) * 0.1,
               "m.up_proj.weight": torch.randn(inter, hidden, generator=g) * 0.1,
               "m.down_proj.weight": torch.randn(hidden, inter, generator=g) * 0.1}
    ffn = FEED_FORWARDS.find("swiglu")({"hidden_size": hidden, "intermediate_size": inter}, "m", tensors, dtype, DEV)
    round_to = torch.bfloat16 if dtype == torch.bfloat16 else None
    rounded = lambda v: v if round_to is None else v.to(round_to).to(v.dtype)  # noqa: E731
    h = torch.randn(tokens, hidden, generator=g).to(dtype)
    pools, runner = _context(dtype, {}, [])
    ctx = _step(pools, runner, [(0, 0, tokens, 1)])
    residual0 = torch.randn(tokens, hidden, generator=g)
    residual = residual0.to(DEV)
    ffn.forward(ctx, h.to(DEV), residual)
    want = residual0.double() + plain.swiglu(h.double(), *(rounded(tensors[f"m.{n}_proj.weight"].double())
                                                           for n in ("gate", "up", "down")), round_to=round_to)
    assert _rel(residual, want) < LIMIT[dtype]

    # a whole block: the four parts in the pre-norm arrangement, on one sequence
    heads, kv_heads, d = 2, 1, 32
    attention = {k.replace("a.", "L.att."): v for k, v in _attention_tensors(hidden, heads, kv_heads, d, True, 5).items()}
    block_tensors = dict(attention)
    block_tensors.update({k.replace("m.", "L.ffn."): v for k, v in tensors.items()})
    block_tensors["L.n1.weight"] = 1 + 0.1 * torch.randn(hidden, generator=g)
    block_tensors["L.n2.weight"] = 1 + 0.1 * torch.randn(hidden, generator=g)
    norm = PartSpec("rmsnorm", {"size": hidden, "eps": 1e-5})
    spec = LayerSpec(
        block="prenorm", prefix="L", parts={"mixer_norm": norm, "ffn_norm": norm,
        "mixer": PartSpec("gqa_attention", {
            "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": d, "qkv_bias": True,
            "window": None, "softmax_scale": 1 / math.sqrt(d),
            "position": PartSpec("rope_neox", {"head_dim": d, "theta": 10000.0, "max_positions": 512})}),
        "ffn": PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inter})},
        names={"mixer_norm": "n1", "mixer": "att", "ffn_norm": "n2", "ffn": "ffn"})
    block_cls = BLOCKS.find("prenorm")
    assert set(block_cls.schema(spec)) == set(block_tensors)
    block = block_cls(spec, block_tensors, dtype, DEV)
    pools, runner = _context(dtype, {0: block.cache_request()}, [])
    ctx = _step(pools, runner, [(0, 0, tokens, 1)])
    x0 = torch.randn(tokens, hidden, generator=g)
    x = x0.to(DEV)
    block.forward(ctx, x, pools.views[0], True)
    xd = x0.double()
    hn = rounded(plain.rms_norm(xd, block_tensors["L.n1.weight"].double(), 1e-5))
    xd = xd + _plain_attention_part({k.replace("L.att.", "a."): v for k, v in attention.items()}, hn, heads, kv_heads,
                                    d, 10000.0, None, True, round_to)
    hn = rounded(plain.rms_norm(xd, block_tensors["L.n2.weight"].double(), 1e-5))
    xd = xd + plain.swiglu(hn, *(rounded(tensors[f"m.{n}_proj.weight"].double()) for n in ("gate", "up", "down")),
                           round_to=round_to)
    assert _rel(x, xd) < LIMIT[dtype]


# ---------------------------------------------------------------------------------------
# toy parts, defined here, registered here
# ---------------------------------------------------------------------------------------
def _register_toys():
    import toy_parts

    toy_parts.register()


def _toy_plugin():
    import toy_parts

    return toy_parts.__file__


def _toy_folder(architecture, dtype, extra=None):
    from vipera_rs_b200.engine import write_random_model

    config = dict(helpers.TINY_A, architectures=[architecture])
    config.update(extra or {})
    folder = tempfile.mkdtemp(prefix=f"vipera_{architecture}_")
    write_random_model(folder, config, seed=9, dtype=dtype)
    return folder


def _plain_toy_state(folder, tokens):
    """The toy architecture by the plain functions: layer 0's mixer is the running mean."""
    config, weights = plain.read_config(folder), plain.read_weights(folder)
    n = len(tokens)
    x = plain.embedding(weights["model.embed_tokens.weight"], tokens, torch.float64)
    h = plain.rms_norm(x, weights["model.layers.0.input_layernorm.weight"], config["eps"])
    means = torch.cumsum(h, dim=0) / torch.arange(1, n + 1, dtype=torch.float64)[:, None]
    x = x + means @ weights["model.layers.0.self_attn.mix.weight"].double().T
    p = "model.layers.0."
    h = plain.rms_norm(x, weights[p + "post_attention_layernorm.weight"], config["eps"])
    x = x + plain.swiglu(h, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                         weights[p + "mlp.down_proj.weight"])
    # layer 1 is an ordinary Qwen2 layer: reuse the plain model on a one-layer view of the weights
    sin, cos = plain.rope_angles(range(n), config["head_dim"], config["rope_base"])
    p = "model.layers.1."
    h = plain.rms_norm(x, weights[p + "input_layernorm.weight"], config["eps"])
    heads, kv_heads, d = config["heads"], config["kv_heads"], config["head_dim"]
    proj = lambda name: h @ weights[p + f"self_attn.{name}.weight"].double().T + weights[p + f"self_attn.{name}.bias"].double()  # noqa: E731
    q = plain.rope_neox(proj("q_proj").view(n, heads, d), sin, cos)
    k = plain.rope_neox(proj("k_proj").view(n, kv_heads, d), sin, cos)
    v = proj("v_proj").view(n, kv_heads, d)
    x = x + plain.attention(q, k, v).reshape(n, heads * d) @ weights[p + "self_attn.o_proj.weight"].double().T
    h = plain.rms_norm(x, weights[p + "post_attention_layernorm.weight"], config["eps"])
    x = x + plain.swiglu(h, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                         weights[p + "mlp.down_proj.weight"])
    h = plain.rms_norm(x, weights["model.norm.weight"], config["eps"])
    return (h @ weights["model.embed_tokens.weight"].double().T).numpy()


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    """A mixer with per-request state, defined in this file: replayed whole, in portions beside
    another request, and token by token, it gives the plain result; and through the engine, with
    so few pages that a request starts over, its state starts over with it."""
    _register_toys()
    from vipera_rs_b200 import Engine, SamplingParams
    from vipera_rs_b200.parts import FixedState

    folder = _toy_folder("ToyStateLM", "float32")
    vocab = helpers.TINY_A["vocab_size"]
    requests = {"a": helpers.random_tokens(vocab, 60, 1), "b": helpers.random_tokens(vocab, 41, 2)}
    builder = helpers.TraceBuilder()
    builder.step([("a", requests["a"][:17], range(17)), ("b", requests["b"][:5], range(5))])
    builder.step([("a", requests["a"][17:19], range(2)), ("b", requests["b"][5:41], range(36))], end=["b"])
    builder.step([("a", requests["a"][19:50], range(31))])
    for position in range(50, 60):
        builder.step([("a", requests["a"][position:position + 1], [0])], end=["a"] if position == 59 else [])
    outputs = helpers.run_trace(folder, "float32", builder.steps, max_tokens=128, page_size=16,
                                env_extra={"VIPERA_PLUGINS": _toy_plugin()})
    reference = {name: _plain_toy_state(folder, tokens) for name, tokens in requests.items()}
    worst = helpers.compare(outputs, builder, reference, 1e-4, "toy state model")
    assert worst < 1e-4

    engine = Engine(folder, dtype="float32", page_size=16, num_pages=9, max_num_seqs=3, max_tokens_per_step=32)
    assert any(isinstance(r, FixedState) for r in engine.model.cache_requests.values())
    assert not engine.model.graph_safe
    assert not engine.lookahead   # a step launched ahead and dropped would move the mixer's state twice
    prompts = [helpers.random_tokens(vocab, n, 10 + n) for n in (30, 45, 20)]
    results = engine.generate(prompts, SamplingParams(max_new_tokens=30))
    assert sum(r.preemptions for r in results) >= 1
    for prompt, result in zip(prompts, results):
        logits = _plain_toy_state(folder, prompt + result.tokens[:-1])
        for index, token in enumerate(result.tokens):
            row = logits[len(prompt) - 1 + index]
            assert row.max() - row[token] <= 1e-4 * np.abs(row).max()
    assert engine.pools.audit() == "" and engine.stats()["sequences"] == 0


def _plain_toy_routed(folder, tokens):
    """Layer 0's feed-forward sends every token to one expert; the rest is the plain model."""
    config, weights = plain.read_config(folder), plain.read_weights(folder)
    n = len(tokens)
    heads, kv_heads, d = config["heads"], config["kv_heads"], config["head_dim"]
    sin, cos = plain.rope_angles(range(n), d, config["rope_base"])
    x = plain.embedding(weights["model.embed_tokens.weight"], tokens, torch.float64)
    for layer in range(2):
        p = f"model.layers.{layer}."
        h = plain.rms_norm(x, weights[p + "input_layernorm.weight"], config["eps"])
        proj = lambda name: h @ weights[p + f"self_attn.{name}.weight"].double().T + weights[p + f"self_attn.{name}.bias"].double()  # noqa: E731
        q = plain.rope_neox(proj("q_proj").view(n, heads, d), sin, cos)
        k = plain.rope_neox(proj("k_proj").view(n, kv_heads, d), sin, cos)
        v = proj("v_proj").view(n, kv_heads, d)
        x = x + plain.attention(q, k, v).reshape(n, heads * d) @ weights[p + "self_attn.o_proj.weight"].double().T
        h = plain.rms_norm(x, weights[p + "post_attention_layernorm.weight"], config["eps"])
        if layer == 0:
            scores = h @ weights[p + "mlp.router.weight"].double().T
            out = torch.zeros_like(x)
            for t in range(n):
                e = int(scores[t].argmax())
                up = weights[p + f"mlp.experts.{e}.up.weight"].double()
                down = weights[p + f"mlp.experts.{e}.down.weight"].double()
                out[t] = torch.relu(h[t] @ up.T) @ down.T
            x = x + out
        else:
            x = x + plain.swiglu(h, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                                 weights[p + "mlp.down_proj.weight"])
    h = plain.rms_norm(x, weights["model.norm.weight"], config["eps"])
    return (h @ weights["model.embed_tokens.weight"].double().T).numpy()


def test_toy_feed_forward_with_routing_is_registered_built_and_stepped():
    """A feed-forward that routes tokens to experts, defined in the tests and chosen for one
    layer only: in portions beside another request and token by token (from a captured graph:
    the part stays on the device) it gives the plain result."""
    _register_toys()
    folder = _toy_folder("ToyRoutedLM", "float32")
    vocab = helpers.TINY_A["vocab_size"]
    requests = {"a": helpers.random_tokens(vocab, 52, 5), "b": helpers.random_tokens(vocab, 30, 6)}
    builder = helpers.TraceBuilder()
    builder.step([("a", requests["a"][:20], range(20)), ("b", requests["b"][:7], range(7))])
    builder.step([("a", requests["a"][20:22], range(2)), ("b", requests["b"][7:30], range(23))], end=["b"])
    builder.step([("a", requests["a"][22:40], range(18))])
    for position in range(40, 52):
        builder.step([("a", requests["a"][position:position + 1], [0])], end=["a"] if position == 51 else [])
    outputs = helpers.run_trace(folder, "float32", builder.steps, max_tokens=128, page_size=16,
                                env_extra={"VIPERA_PLUGINS": _toy_plugin()})
    reference = {name: _plain_toy_routed(folder, tokens) for name, tokens in requests.items()}
    worst = helpers.compare(outputs, builder, reference, 1e-4, "toy routed model")
    assert worst < 1e-4


def _plain_toy_arranged(folder, tokens):
    """Layer 0 with four norms and half-weight branches, layer 1 with mixer and feed-forward side
    by side under one norm, embedding rows times three; by the plain functions."""
    config, weights = plain.read_config(folder), plain.read_weights(folder)
    n = len(tokens)
    heads, kv_heads, d, eps = config["heads"], config["kv_heads"], config["head_dim"], config["eps"]
    sin, cos = plain.rope_angles(range(n), d, config["rope_base"])

    def attend(p, h):
        proj = lambda name: h @ weights[p + f"self_attn.{name}.weight"].double().T + weights[p + f"self_attn.{name}.bias"].double()  # noqa: E731
        q = plain.rope_neox(proj("q_proj").view(n, heads, d), sin, cos)
        k = plain.rope_neox(proj("k_proj").view(n, kv_heads, d), sin, cos)
        v = proj("v_proj").view(n, kv_heads, d)
        return plain.attention(q, k, v).reshape(n, heads * d) @ weights[p + "self_attn.o_proj.weight"].double().T

    def feed(p, h):
        return plain.swiglu(h, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                            weights[p + "mlp.down_proj.weight"])

    x = 3.0 * plain.embedding(weights["model.embed_tokens.weight"], tokens, torch.float64)
    p = "model.layers.0."
    branch = attend(p, plain.rms_norm(x, weights[p + "input_layernorm.weight"], eps))
    x = x + 0.5 * plain.rms_norm(branch, weights[p + "post_mixer_norm.weight"], eps)
    branch = feed(p, plain.rms_norm(x, weights[p + "post_attention_layernorm.weight"], eps))
    x = x + 0.5 * plain.rms_norm(branch, weights[p + "post_ffn_norm.weight"], eps)
    p = "model.layers.1."
    h = plain.rms_norm(x, weights[p + "input_layernorm.weight"], eps)
    x = x + attend(p, h) + feed(p, h)
    h = plain.rms_norm(x, weights["model.norm.weight"], eps)
    return (h @ weights["model.embed_tokens.weight"].double().T).numpy()


def test_other_arrangements_of_a_layer_need_a_block_class_only():
    """A layer with four norms, a layer whose mixer and feed-forward run side by side, and scaled
    embedding rows: two block arrangements registered from the tests and one field of the model's
    description; replayed in portions beside another request and token by token."""
    _register_toys()
    from vipera_rs_b200.config import BLOCKS, load_config, read_config_json

    folder = _toy_folder("ToyArrangedLM", "float32")
    names = set(plain.read_weights(folder))
    assert "model.layers.0.post_mixer_norm.weight" in names and "model.layers.0.post_ffn_norm.weight" in names
    assert "model.layers.1.post_attention_layernorm.weight" not in names   # the parallel layer has one norm
    assert "toy_sandwich" in BLOCKS and "toy_parallel" in BLOCKS
    vocab = helpers.TINY_A["vocab_size"]
    requests = {"a": helpers.random_tokens(vocab, 52, 7), "b": helpers.random_tokens(vocab, 30, 8)}
    builder = helpers.TraceBuilder()
    builder.step([("a", requests["a"][:20], range(20)), ("b", requests["b"][:7], range(7))])
    builder.step([("a", requests["a"][20:22], range(2)), ("b", requests["b"][7:30], range(23))], end=["b"])
    builder.step([("a", requests["a"][22:40], range(18))])
    for position in range(40, 52):
        builder.step([("a", requests["a"][position:position + 1], [0])], end=["a"] if position == 51 else [])
    outputs = helpers.run_trace(folder, "float32", builder.steps, max_tokens=128, page_size=16,
                                env_extra={"VIPERA_PLUGINS": _toy_plugin()})
    reference = {name: _plain_toy_arranged(folder, tokens) for name, tokens in requests.items()}
    worst = helpers.compare(outputs, builder, reference, 1e-4, "toy arranged model")
    assert worst < 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_runs_a_layer_twice_and_shares_a_cache(dtype):
    _register_toys()
    folder = _toy_folder("ToySharedLM", dtype)
    vocab = helpers.TINY_A["vocab_size"]
    tokens = helpers.random_tokens(vocab, 50, 4)
    builder = helpers.TraceBuilder()
    builder.step([("s", tokens[:23], range(23))])
    builder.step([("s", tokens[23:25], range(2))])
    for position in range(25, 50):
        builder.step([("s", tokens[position:position + 1], [0])], end=["s"] if position == 49 else [])
    outputs = helpers.run_trace(folder, dtype, builder.steps, max_tokens=64, page_size=16,
                                env_extra={"VIPERA_PLUGINS": _toy_plugin()})
    config, weights = plain.read_config(folder), plain.read_weights(folder)
    round_to = torch.bfloat16 if dtype == "bfloat16" else None
    want = plain.forward(config, weights, tokens, round_to=round_to,
                         schedule=[(0, 0, True), (0, 1, True), (1, 0, False)]).numpy()
    helpers.compare(outputs, builder, {"s": want}, 1e-4 if dtype == "float32" else 1e-2, f"shared schedule {dtype}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_position_encoding_runs_unfused(dtype):
    """An encoding the kernels do not know: the attention part applies it through apply()."""
    _register_toys()
    from vipera_rs_b200.config import MIXERS, PartSpec

    hidden, heads, kv_heads, d, n = 64, 2, 1, 32, 40
    tensors = _attention_tensors(hidden, heads, kv_heads, d, True, seed=11)
    tensors["a.shift.weight"] = torch.randn(128, d) * 0.3
    params = {"hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": d, "qkv_bias": True,
              "window": None, "softmax_scale": 1 / math.sqrt(d),
              "position": PartSpec("toy_learned_shift", {"head_dim": d, "max_positions": 128})}
    mixer = MIXERS.find("gqa_attention")(params, "a", tensors, dtype, DEV)
    torch.manual_seed(2)
    h = torch.randn(n, hidden).to(dtype)
    round_to = torch.bfloat16 if dtype == torch.bfloat16 else None
    rounded = lambda v: v if round_to is None else v.to(round_to).to(v.dtype)  # noqa: E731
    hd = h.double()
    project = lambda name: hd @ rounded(tensors[f"a.{name}_proj.weight"].double()).T + tensors[f"a.{name}_proj.bias"].double()  # noqa: E731
    shift = tensors["a.shift.weight"].double()[:n][:, None, :]
    q = rounded(project("q").view(n, heads, d) + shift)
    k = rounded(project("k").view(n, kv_heads, d) + shift)
    v = rounded(project("v").view(n, kv_heads, d))
    want = rounded(plain.attention(q, k, v).reshape(n, heads * d)) @ rounded(tensors["a.o_proj.weight"].double()).T
    pools, runner = _context(dtype, {0: mixer.cache_request()}, [])
    got = torch.zeros(n, hidden, dtype=torch.float64)
    done = 0
    for count in (13, 2, 1, 24):
        entries = [(0, done, count, 1 if done == 0 else 0)]
        ctx = _step(pools, runner, entries)
        residual = torch.zeros(count, hidden, device=DEV)
        mixer.forward(ctx, h[done:done + count].to(DEV), residual, pools.views[0], True)
        got[done:done + count] = residual.double().cpu()
        _commit(pools, entries)
        done += count
    assert _rel(got, want) < LIMIT[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_interleaved_rotary_encoding_is_a_registered_kind(dtype):
    """Rotary positions with the other pairing (values 2i and 2i + 1 turn together): a registered
    position encoding the fused endings do not know, so the attention part runs it through the
    rotation kernel behind the q/k/v product; in portions and token by token against the plain
    rotation of those pairs."""
    _pkg()
    from vipera_rs_b200.config import MIXERS, POSITION_ENCODINGS, PartSpec

    assert "rope_interleaved" in POSITION_ENCODINGS
    hidden, heads, kv_heads, d, n, theta = 64, 2, 1, 32, 45, 10000.0
    tensors = _attention_tensors(hidden, heads, kv_heads, d, True, seed=13)
    params = {"hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": d, "qkv_bias": True,
              "window": None, "softmax_scale": 1 / math.sqrt(d),
              "position": PartSpec("rope_interleaved", {"head_dim": d, "theta": theta, "max_positions": 128})}
    mixer = MIXERS.find("gqa_attention")(params, "a", tensors, dtype, DEV)
    torch.manual_seed(3)
    h = torch.randn(n, hidden).to(dtype)
    round_to = torch.bfloat16 if dtype == torch.bfloat16 else None
    rounded = lambda v: v if round_to is None else v.to(round_to).to(v.dtype)  # noqa: E731
    hd = h.double()
    project = lambda name: hd @ rounded(tensors[f"a.{name}_proj.weight"].double()).T + tensors[f"a.{name}_proj.bias"].double()  # noqa: E731
    sin, cos = plain.rope_angles(range(n), d, theta)

    def turn(x):   # pairs (2i, 2i + 1) by the angle of index i
        even, odd = x[..., 0::2], x[..., 1::2]
        s, c = sin.double()[:, None, :], cos.double()[:, None, :]
        out = torch.empty_like(x)
        out[..., 0::2] = even * c - odd * s
        out[..., 1::2] = even * s + odd * c
        return out

    q = rounded(turn(project("q").view(n, heads, d)))
    k = rounded(turn(project("k").view(n, kv_heads, d)))
    v = rounded(project("v").view(n, kv_heads, d))
    want = rounded(plain.attention(q, k, v).reshape(n, heads * d)) @ rounded(tensors["a.o_proj.weight"].double()).T
    pools, runner = _context(dtype, {0: mixer.cache_request()}, [])
    got = torch.zeros(n, hidden, dtype=torch.float64)
    done = 0
    for count in (17, 2, 1, 1, 24):
        entries = [(0, done, count, 1 if done == 0 else 0)]
        ctx = _step(pools, runner, entries)
        residual = torch.zeros(count, hidden, device=DEV)
        mixer.forward(ctx, h[done:done + count].to(DEV), residual, pools.views[0], True)
        got[done:done + count] = residual.double().cpu()
        _commit(pools, entries)
        done += count
    assert _rel(got, want) < LIMIT[dtype]


def test_guard_regions_beside_the_pools_show_a_stray_write():
    """Every pool lies between two guard regions; the audit the tests end with reads them."""
    _pkg()
    from vipera_rs_b200.parts import PagedKV

    pools, _ = _context(torch.bfloat16, {0: PagedKV(2, 64, None), 1: PagedKV(1, 128, 40)}, [])
    assert len(pools.pool_tensors) == 2 and pools.audit() == "" and pools.guards_intact()
    pools.poison()
    assert pools.audit() == ""                      # filling every page touches no guard
    pools.pool_tensors[1].view(-1)[-1:].fill_(3.0)  # the last value of a pool is still the pool's
    assert pools.audit() == ""
    end = pools._guards[3]
    saved = end[:1].clone()
    end[:1].fill_(3.0)                              # one value past the end of the second pool
    assert "guard" in pools.audit()
    end[:1].copy_(saved)
    assert pools.audit() == ""

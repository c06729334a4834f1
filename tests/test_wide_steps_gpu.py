"""Steps of many entries: 40 and 64 requests decoding at once through the entry point, and one
replayed step of 48 single-token entries, held to the plain implementation.  These run what the
small batches of the other tests do not: products with tokens on the 128-row side from 33
tokens on, the split-key attention at many entries with the split count chosen there, captured
graphs of 64 entries and graphs padded from 40 to 64, and steps with dozens of portions."""
import functools
import tempfile

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain
from helpers import TraceBuilder

pytestmark = pytest.mark.gpu

SHAPE_1P5B_2_LAYERS = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 1536,
    "num_attention_heads": 12, "num_key_value_heads": 2, "intermediate_size": 8960, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 32768,
}


@functools.lru_cache(maxsize=None)
def _wide_folder():
    import vipera_rs_b200  # noqa: F401
    from vipera_rs_b200.engine import write_random_model

    path = tempfile.mkdtemp(prefix="vipera_wide_")
    write_random_model(path, SHAPE_1P5B_2_LAYERS, 78, "bfloat16")
    return path


def _check_all_greedy(folder, prompts, results, dtype, new_tokens):
    config, weights = helpers.plain_model(folder)
    round_to = torch.bfloat16 if dtype == "bfloat16" else None
    limit = 1e-4 if dtype == "float32" else 2e-2
    for index, (prompt, result) in enumerate(zip(prompts, results)):
        assert result.finish == "length" and len(result.tokens) == new_tokens
        logits = plain.forward(config, weights, list(prompt) + result.tokens[:-1], dtype=torch.float64,
                               round_to=round_to).numpy()
        for place, token in enumerate(result.tokens):
            row = logits[len(prompt) - 1 + place]
            margin = float(row.max() - row[token])
            assert margin <= limit * float(np.abs(row).max()), (
                f"request {index}, token {place}: engine chose {token}, plain prefers {int(row.argmax())} by {margin}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("count", [40, 64])
def test_many_requests_decode_at_once(count, dtype):
    """`count` prompts of 3 to 40 tokens, all admitted at once, 14 tokens each: steps with dozens
    of portions, then decode steps of `count` entries (a graph of 64 entries; padded for 40)."""
    from vipera_rs_b200 import Engine, SamplingParams

    folder = helpers.model_folder("A", dtype)
    vocab = helpers.CONFIGS["A"]["vocab_size"]
    rng = np.random.default_rng(count)
    prompts = [helpers.random_tokens(vocab, int(rng.integers(3, 41)), 1000 + i) for i in range(count)]
    engine = Engine(folder, dtype=dtype, page_size=16, ctx=64, max_num_seqs=count, max_tokens_per_step=512,
                    max_portion=24)
    results = engine.generate(prompts, SamplingParams(max_new_tokens=14))
    _check_all_greedy(folder, prompts, results, dtype, 14)
    stats = engine.stats()
    assert stats["entries_per_step"] > count / 2 and stats["graph_steps"] >= 10
    assert engine.pools.audit() == ""


def test_forty_requests_on_the_benchmarks_layer_sizes():
    """The same at the layer sizes the benchmark measures (two layers of them): tokens-as-rows
    products from 33 tokens on, the split-key attention at 40 entries of 2 KV heads."""
    from vipera_rs_b200 import Engine, SamplingParams

    folder = _wide_folder()
    vocab = SHAPE_1P5B_2_LAYERS["vocab_size"]
    rng = np.random.default_rng(5)
    prompts = [helpers.random_tokens(vocab, int(rng.integers(2, 30)), 2000 + i) for i in range(40)]
    engine = Engine(folder, dtype="bfloat16", page_size=16, ctx=48, max_num_seqs=40, max_tokens_per_step=1024)
    results = engine.generate(prompts, SamplingParams(max_new_tokens=6))
    _check_all_greedy(folder, prompts, results, "bfloat16", 6)
    assert engine.pools.audit() == ""


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_replayed_step_of_48_single_tokens(dtype):
    """48 live requests: prompts in steps of a dozen portions, then three steps in which each of
    the 48 brings one token and wants its logits; every row against the plain logits."""
    folder = helpers.model_folder("B", dtype)
    vocab = helpers.CONFIGS["B"]["vocab_size"]
    rng = np.random.default_rng(48)
    requests = {f"r{i}": helpers.random_tokens(vocab, int(rng.integers(6, 50)), 3000 + i) for i in range(48)}
    builder = TraceBuilder()
    names = list(requests)
    for first in range(0, 48, 12):                      # prompts, all but the last three tokens
        builder.step([(name, requests[name][:-3], [len(requests[name]) - 4]) for name in names[first:first + 12]])
    for back in (3, 2, 1):
        builder.step([(name, requests[name][-back:len(requests[name]) - back + 1], [0]) for name in names],
                     end=names if back == 1 else [])
    page = 32
    pages = sum(-(-len(tokens) // page) for tokens in requests.values())
    outputs = helpers.run_trace(folder, dtype, builder.steps, max_tokens=pages * page, page_size=page, max_live=48)
    round_to = torch.bfloat16 if dtype == "bfloat16" else None
    reference = {name: helpers.plain_logits(folder, tokens, round_to) for name, tokens in requests.items()}
    worst = helpers.compare(outputs, builder, reference, 1e-4 if dtype == "float32" else 1e-2, f"48 entries {dtype}")
    print(f"48 single-token entries, {dtype}: worst relative error {worst:.3e}")

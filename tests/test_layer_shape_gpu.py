"""The layer sizes of the model the benchmark measures (Qwen2.5-1.5B: hidden 1536, 12 query
heads on 2 KV heads of 128, intermediate 8960, vocabulary 151936, tied output matrix), with
two layers so that the plain implementation stays quick: the kernels run at the very sizes
they are tuned for (the tcgen05 products with 17920 and 151936 rows and an inner size of 8960,
the fused q/k/v ending, the tcgen05 attention, the small-token kernels) and are held to the
plain implementation under the same cuts as the tiny models: whole prompt, decode steps,
portions, and portions beside decode tokens with pages that are used again."""
import functools
import json
import os
import tempfile

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain
from helpers import TraceBuilder

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 1536,
    "num_attention_heads": 12, "num_key_value_heads": 2, "intermediate_size": 8960, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 32768, "use_sliding_window": False, "sliding_window": 32768,
    "max_window_layers": 28,
}


@functools.lru_cache(maxsize=None)
def _folder():
    import vipera_rs_b200  # noqa: F401
    from vipera_rs_b200.engine import write_random_model

    path = tempfile.mkdtemp(prefix="vipera_layer_shape_")
    write_random_model(path, CONFIG, 77, "bfloat16")
    return path


def _trace(vocab):
    builder = TraceBuilder()
    requests = {
        "long": helpers.random_tokens(vocab, 230, 1),      # more than 192 tokens: tokens on the 128-row side
        "cut": helpers.random_tokens(vocab, 120, 2),
        "short": helpers.random_tokens(vocab, 21, 3),
    }
    long, cut, short = requests["long"], requests["cut"], requests["short"]
    builder.step([("long", long[:214], [0, 100, 191, 213])])
    builder.step([("cut", cut[:48], [47]), ("long", long[214:215], [0])])
    builder.step([("cut", cut[48:65], [16]), ("long", long[215:216], [0]), ("short", short[:20], [19])])
    builder.step([("cut", cut[65:70], [4]), ("long", long[216:217], [0]), ("short", short[20:21], [0])], end=["short"])
    builder.step([("cut", cut[70:118], [47]), ("long", long[217:218], [0])])
    for position in range(218, 230):
        entries = [("long", long[position:position + 1], [0])]
        if position < 220:
            entries.append(("cut", cut[position - 100:position - 99], [0]))
        builder.step(entries, end=["long"] if position == 229 else (["cut"] if position == 219 else []))
    return builder, requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_benchmarks_layer_sizes_match_plain(dtype):
    folder = _folder()
    vocab = CONFIG["vocab_size"]
    builder, requests = _trace(vocab)
    outputs = helpers.run_trace(folder, dtype, builder.steps, max_tokens=448, page_size=16, timeout=1200)
    config, weights = plain.read_config(folder), plain.read_weights(folder)
    round_to = torch.bfloat16 if dtype == "bfloat16" else None
    reference = {name: plain.forward(config, weights, tokens, dtype=torch.float64, round_to=round_to).numpy()
                 for name, tokens in requests.items()}
    tolerance = 1e-4 if dtype == "float32" else 1e-2
    worst = helpers.compare(outputs, builder, reference, tolerance, f"1.5B layer sizes {dtype}")
    print(f"1.5B layer sizes, {dtype}: worst relative error {worst:.3e}")


def test_a_long_portion_at_the_benchmarks_layer_sizes_matches_plain():
    """A prompt of 1,700 tokens in one step and a few decode steps behind it, bfloat16: at this
    length the feed-forward products run on pairs of blocks (tiles of 256 tokens), the q/k/v
    product ends inside the product kernel and the attention of portions walks fourteen key
    tiles; the tiny models never get there."""
    folder = _folder()
    vocab = CONFIG["vocab_size"]
    tokens = helpers.random_tokens(vocab, 1704, 11)
    builder = TraceBuilder()
    builder.step([("p", tokens[:1700], [0, 127, 128, 1023, 1699])])
    for position in range(1700, 1704):
        builder.step([("p", tokens[position:position + 1], [0])], end=["p"] if position == 1703 else [])
    outputs = helpers.run_trace(folder, "bfloat16", builder.steps, max_tokens=1728, page_size=16, timeout=1200)
    config, weights = plain.read_config(folder), plain.read_weights(folder)
    reference = {"p": plain.forward(config, weights, tokens, dtype=torch.float64, round_to=torch.bfloat16).numpy()}
    worst = helpers.compare(outputs, builder, reference, 1e-2, "1.5B layer sizes, long portion")
    print(f"1.5B layer sizes, 1,700-token portion: worst relative error {worst:.3e}")

"""Trace replay against the plain implementation, in 32-bit and in bfloat16: each request
alone and whole; most of it in one step and the last 32 tokens one by one; in portions of
changing size down to two tokens; and mixed, up to four live requests, with so few pages
that they are used again."""
import numpy as np
import pytest
import torch

import helpers
from helpers import TraceBuilder

pytestmark = pytest.mark.gpu

PAGE = {"A": 16, "B": 32, "C": 64, "A_stated": 16, "B_stated": 32}
LENGTHS = {"A": [1, 7, 33, 64, 200], "B": [5, 100, 257], "C": [2, 50, 130],
           "A_stated": [1, 7, 33, 64], "B_stated": [5, 100, 257]}
FP32_TOL = 1e-4
BF16_TOL = 1e-2  # of the request's largest |logit|; bfloat16 keeps 8 bits of mantissa

PORTIONS = [48, 17, 5, 3, 2, 2, 31, 64, 2, 7, 19, 2, 90]


def build_trace(name, vocab):
    """One trace holding all four regimes, and the tokens of every request in it."""
    builder = TraceBuilder()
    requests = {}
    page = PAGE[name]
    # 1. each request alone and whole, every position wanted
    for index, length in enumerate(LENGTHS[name]):
        rid = f"whole{index}"
        requests[rid] = helpers.random_tokens(vocab, length, 100 + index)
        builder.step([(rid, requests[rid], range(length))], end=[rid])
    # 2. most of it in one step, the last 32 tokens one by one
    for index, length in enumerate(LENGTHS[name]):
        if length <= 33:
            continue
        rid = f"tail{index}"
        tokens = requests[rid] = helpers.random_tokens(vocab, length, 200 + index)
        bulk = length - 32
        builder.step([(rid, tokens[:bulk], [bulk - 1])])
        for position in range(bulk, length):
            last = position == length - 1
            builder.step([(rid, tokens[position:position + 1], [0])], end=[rid] if last else [])
    # 3. portions of changing size, down to two tokens
    for index, length in enumerate(LENGTHS[name]):
        if length < 8:
            continue
        rid = f"cut{index}"
        tokens = requests[rid] = helpers.random_tokens(vocab, length, 300 + index)
        done, turn = 0, index
        while done < length:
            size = min(PORTIONS[turn % len(PORTIONS)], length - done)
            if length - done - size == 1:  # never leave a single token: portions have two at least
                size += 1
            turn += 1
            last = done + size == length
            builder.step([(rid, tokens[done:done + size], range(size))], end=[rid] if last else [])
            done += size
    # 4. mixed: four live requests, portions of some beside decode tokens of others
    lengths = [90, 61, 130, 47, 75, 38]
    for index, length in enumerate(lengths):
        requests[f"mix{index}"] = helpers.random_tokens(vocab, length, 400 + index)
    state = {f"mix{index}": 0 for index in range(len(lengths))}
    waiting = [f"mix{index}" for index in range(len(lengths))]
    live = []
    turn = 0
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        entries, ended = [], []
        for slot, rid in enumerate(list(live)):
            tokens, done = requests[rid], state[rid]
            prompt = len(tokens) - 12  # the last 12 tokens go one by one
            if done < prompt:
                size = min([23, 2, 40, 9][(turn + slot) % 4], prompt - done)
                if (turn + slot) % 5 == 4:
                    continue  # left out of this step, goes on later
            else:
                size = 1
            entries.append((rid, tokens[done:done + size], range(size)))
            state[rid] = done + size
            if state[rid] == len(tokens):
                ended.append(rid)
                live.remove(rid)
        if entries:
            builder.step(entries, end=ended)
        turn += 1
    # pages for the four longest requests of the mixed part at once, each rounded up to a page
    rounded = sorted(((length + page - 1) // page * page for length in lengths), reverse=True)
    longest = max((max(LENGTHS[name]) + page - 1) // page * page, sum(rounded[:4]))
    return builder, requests, longest


@pytest.mark.parametrize("name", ["A", "B", "C", "A_stated", "B_stated"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_matches_plain(name, dtype):
    folder = helpers.model_folder(name, dtype)
    vocab = helpers.CONFIGS[name]["vocab_size"]
    builder, requests, max_tokens = build_trace(name, vocab)
    outputs = helpers.run_trace(folder, dtype, builder.steps, max_tokens=max_tokens, page_size=PAGE[name])
    round_to = torch.bfloat16 if dtype == "bfloat16" else None
    reference = {rid: helpers.plain_logits(folder, tokens, round_to) for rid, tokens in requests.items()}
    tolerance = FP32_TOL if dtype == "float32" else BF16_TOL
    worst = helpers.compare(outputs, builder, reference, tolerance, f"tiny {name} {dtype}")
    print(f"tiny {name} {dtype}: worst relative error {worst:.3e} over {len(builder.steps)} steps")

"""Generation through the public entry point on the GPU, held to the plain implementation."""
import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu


def _engine(name, dtype, **kwargs):
    from vipera_rs_b200 import Engine

    folder = helpers.model_folder(name, dtype)
    return folder, Engine(folder, dtype=dtype, device="cuda:0", **kwargs)


def _check_greedy(folder, prompt, produced, dtype):
    """Each produced token is the plain implementation's best at its place (or ties it
    within rounding), given the tokens produced before it."""
    round_to = torch.bfloat16 if dtype == "bfloat16" else None
    logits = helpers.plain_logits(folder, list(prompt) + list(produced[:-1]), round_to)
    limit = 1e-4 if dtype == "float32" else 2e-2
    for index, token in enumerate(produced):
        row = logits[len(prompt) - 1 + index]
        margin = float(row.max() - row[token])
        assert margin <= limit * float(np.abs(row).max()), (
            f"token {index}: engine chose {token}, plain prefers {int(row.argmax())} by {margin}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_tiny_a(dtype):
    from vipera_rs_b200 import SamplingParams

    folder, engine = _engine("A", dtype, page_size=16, ctx=128, max_num_seqs=4)
    vocab = helpers.CONFIGS["A"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 500 + n) for n in (1, 7, 33, 64)]
    results = engine.generate(prompts, SamplingParams(max_new_tokens=16))
    for prompt, result in zip(prompts, results):
        assert result.finish == "length" and len(result.tokens) == 16
        _check_greedy(folder, prompt, result.tokens, dtype)
    stats = engine.stats()
    # only the pages kept for requests that begin the same way are still in use
    assert stats["kv_used_pages"] == stats["kv_kept_pages"] == 6 and stats["sequences"] == 0
    assert engine.pools.audit() == ""


def test_batched_equals_alone_and_seed_replays():
    """A request's tokens do not depend on what else runs beside it, and the same seed gives
    the same tokens (crates/vipera-runtime/src/engine.rs:1770-1806, 1906-1941)."""
    from vipera_rs_b200 import SamplingParams

    folder, engine = _engine("B", "float32", page_size=32, ctx=512, max_num_seqs=3, max_tokens_per_step=48)
    vocab = helpers.CONFIGS["B"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 600 + n) for n in (5, 100, 257)]
    params = SamplingParams(max_new_tokens=24, temperature=0.8, seed=1234)
    together = engine.generate(prompts, params)
    alone = [engine.generate([prompt], params)[0] for prompt in prompts]
    for a, b in zip(together, alone):
        assert a.tokens == b.tokens
    again = engine.generate(prompts[:1], params)[0]
    assert again.tokens == together[0].tokens
    other = engine.generate(prompts[:1], SamplingParams(max_new_tokens=24, temperature=0.8, seed=4321))[0]
    assert other.tokens != together[0].tokens
    assert engine.pools.audit() == ""


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_few_pages_preempt_and_recompute(dtype):
    """With too few pages for all requests at once, the one admitted last is put back and
    computed again; every request still gets the tokens it gets alone."""
    from vipera_rs_b200 import SamplingParams

    folder, engine = _engine("A", dtype, page_size=16, num_pages=14, max_num_seqs=4, max_tokens_per_step=64)
    vocab = helpers.CONFIGS["A"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 700 + n) for n in (40, 50, 60, 30)]
    params = SamplingParams(max_new_tokens=40)
    results = engine.generate(prompts, params)
    assert sum(r.preemptions for r in results) >= 1
    for prompt, result in zip(prompts, results):
        assert len(result.tokens) == 40
        _check_greedy(folder, prompt, result.tokens, dtype)
    assert engine.pools.audit() == ""
    assert engine.stats()["kv_used_pages"] == engine.stats()["kv_kept_pages"]   # nothing but pages kept for reuse
    assert sum(r.reused_tokens for r in results if r.preemptions) > 0             # who was put back found its pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_the_first_tokens(dtype):
    """A one-token prompt decoded for 300 steps (over many pages, through the decode graphs of
    growing table widths): the first tokens and every later one are the plain implementation's
    choices."""
    from vipera_rs_b200 import SamplingParams

    folder, engine = _engine("A", dtype, page_size=16, ctx=512, max_num_seqs=2)
    prompt = [7]
    result = engine.generate([prompt], SamplingParams(max_new_tokens=300))[0]
    assert len(result.tokens) == 300 and result.finish == "length"
    _check_greedy(folder, prompt, result.tokens, dtype)
    # the same through steps without graphs gives the same tokens
    _, eager = _engine("A", dtype, page_size=16, ctx=512, max_num_seqs=2, decode_graphs=False)
    again = eager.generate([prompt], SamplingParams(max_new_tokens=60))[0]
    if dtype == "float32":
        assert again.tokens == result.tokens[:60]


def test_temperature_sampling_is_the_plain_samplers_on_the_plain_logits():
    """The second tiny configuration's workload as the baseline states it: prompts of 5, 100 and 257
    tokens in portions of 48 beside running decodes, then 24 tokens each at temperature 0.8 with
    a fixed seed.  Every token is what the plain restatement of the reference's sampler draws
    from the plain implementation's logits with the same generator, one draw a token."""
    import plain_sampler
    from vipera_rs_b200 import SamplingParams

    folder, engine = _engine("B_stated", "float32", page_size=32, ctx=512, max_num_seqs=3, max_tokens_per_step=64,
                             max_portion=48)
    vocab = helpers.CONFIGS["B_stated"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 800 + n) for n in (5, 100, 257)]
    seed = 20240
    results = engine.generate(prompts, SamplingParams(max_new_tokens=24, temperature=0.8, seed=seed, eos_ids=[]))
    assert engine.stats()["steps_with_portions"] >= 6
    for prompt, result in zip(prompts, results):
        assert len(result.tokens) == 24
        logits = helpers.plain_logits(folder, list(prompt) + result.tokens[:-1])
        rng = plain_sampler.Rng(seed)
        for index, token in enumerate(result.tokens):
            row = [plain_sampler.f32(float(v)) for v in logits[len(prompt) - 1 + index]]
            want = plain_sampler.temperature(row, 0.8, 40, 0.95, 0.05, rng.next_f64())
            assert token == want, f"prompt of {len(prompt)}: token {index} is {token}, the plain sampler draws {want}"
    assert engine.pools.audit() == ""


def test_sampling_options_through_the_entry_point():
    """Temperature with penalties and a bias on the device gives what the host sampler gives on
    the same logits (checked through determinism and the ban of one token)."""
    from vipera_rs_b200 import SamplingParams

    folder, engine = _engine("C", "float32", page_size=64, ctx=256, max_num_seqs=2)
    vocab = helpers.CONFIGS["C"]["vocab_size"]
    prompt = helpers.random_tokens(vocab, 20, 3)
    greedy = engine.generate([prompt], SamplingParams(max_new_tokens=8))[0].tokens
    banned = greedy[0]
    params = SamplingParams(max_new_tokens=8, temperature=0.0, logit_bias=[(banned, -100.0)])
    other = engine.generate([prompt], params)[0].tokens
    assert other[0] != banned and banned not in other
    sampled = SamplingParams(max_new_tokens=12, temperature=0.9, top_k=0, top_p=0.9, min_p=0.0, seed=5,
                             repetition_penalty=1.2, frequency_penalty=0.3)
    a = engine.generate([prompt], sampled)[0].tokens       # top_k = 0: rows the device hands to the host sampler
    b = engine.generate([prompt], sampled)[0].tokens
    assert a == b and len(a) == 12
    stop = SamplingParams(max_new_tokens=8, eos_ids=[greedy[2]])
    ended = engine.generate([prompt], stop)[0]
    assert ended.finish == "stop" and ended.tokens == greedy[:greedy.index(greedy[2]) + 1]   # the end token is kept


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_seen_before_shares_its_pages(dtype):
    """The pages of a prompt stay known after its request ends; a request that begins with the
    same tokens takes them over instead of computing them (at least one token is computed),
    produces tokens the plain implementation agrees with, and a tiny B model with windowed
    layers (pages given back) does not share at all."""
    from vipera_rs_b200 import SamplingParams

    folder, engine = _engine("A", dtype, page_size=16, num_pages=24, max_num_seqs=2)
    vocab = helpers.CONFIGS["A"]["vocab_size"]
    prompt = helpers.random_tokens(vocab, 75, 900)
    params = SamplingParams(max_new_tokens=10)
    first = engine.generate([prompt], params)[0]
    assert first.reused_tokens == 0 and engine.stats()["kv_kept_pages"] == 4
    again, branch = engine.generate([prompt, prompt[:40] + helpers.random_tokens(vocab, 9, 901)], params)
    assert again.reused_tokens == 64 and again.processed_tokens == 75 - 64 + 9
    assert branch.reused_tokens == 32
    _check_greedy(folder, prompt, again.tokens, dtype)
    _check_greedy(folder, prompt[:40] + helpers.random_tokens(vocab, 9, 901), branch.tokens, dtype)
    if dtype == "float32":
        assert again.tokens == first.tokens
    # without it nothing is kept
    _, plain_engine = _engine("A", dtype, page_size=16, num_pages=24, max_num_seqs=2, prefix_cache=False)
    plain_engine.generate([prompt], params)
    assert plain_engine.generate([prompt], params)[0].reused_tokens == 0
    assert plain_engine.stats()["kv_kept_pages"] == 0
    _, windowed = _engine("B", dtype, page_size=32, ctx=256, max_num_seqs=2)
    assert not windowed.pools.manager.reuse


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_change_no_token(dtype):
    """Greedy decoding with the step after launched before a step's tokens are read: the same
    tokens as without it, also where a request ends on an end token while the step after it
    already runs (that step is dropped), where a request arrives in the middle of decoding,
    and where requests of different lengths end one after the other."""
    from vipera_rs_b200 import SamplingParams

    vocab = helpers.CONFIGS["A"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 900 + n) for n in (3, 20, 41)]
    folder, plain_engine = _engine("A", dtype, page_size=16, ctx=160, max_num_seqs=4, lookahead=False)
    _, ahead_engine = _engine("A", dtype, page_size=16, ctx=160, max_num_seqs=4, lookahead=True)
    lengths = [SamplingParams(max_new_tokens=n) for n in (30, 9, 17)]
    want = plain_engine.generate(prompts, lengths)
    got = ahead_engine.generate(prompts, lengths)
    assert [g.tokens for g in got] == [w.tokens for w in want]
    assert ahead_engine.steps_ahead > 0 and plain_engine.steps_ahead == 0
    _check_greedy(folder, prompts[0], got[0].tokens, dtype)
    # an end token in the middle: the first token the first request produces after its third
    # that it has not produced before
    produced = want[0].tokens
    first = next(i for i in range(3, len(produced)) if produced[i] not in produced[:i])
    stop = SamplingParams(max_new_tokens=30, eos_ids=[produced[first]])
    for engine in (plain_engine, ahead_engine):
        result = engine.generate([prompts[0], prompts[2]], [stop, SamplingParams(max_new_tokens=17)])
        assert result[0].finish == "stop" and result[0].tokens == want[0].tokens[:first + 1]
        assert result[1].tokens == want[2].tokens
    assert ahead_engine.steps_ahead_dropped > 0
    # a request that arrives while another decodes
    request = ahead_engine.add_request(prompts[1], SamplingParams(max_new_tokens=9))
    for _ in range(4):
        ahead_engine.step()
    late = ahead_engine.add_request(prompts[2], SamplingParams(max_new_tokens=17))
    results = {}
    while ahead_engine.has_work():
        for generation in ahead_engine.step().finished:
            results[generation.request] = generation.tokens
    assert results[request] == want[1].tokens and results[late] == want[2].tokens
    # rows drawn with a temperature (and a top-k the device draws alone) are launched ahead too,
    # with the draws their generators hand out next: the same tokens
    sampling = SamplingParams(max_new_tokens=20, temperature=0.9, top_k=50, top_p=0.9, seed=77)
    before = ahead_engine.steps_ahead
    drawn_ahead = ahead_engine.generate(prompts, sampling)
    drawn_plain = plain_engine.generate(prompts, sampling)
    assert [g.tokens for g in drawn_ahead] == [g.tokens for g in drawn_plain]
    assert ahead_engine.steps_ahead > before
    assert ahead_engine.pools.audit() == "" and plain_engine.pools.audit() == ""
    stats = ahead_engine.stats()
    assert stats["sequences"] == 0 and stats["kv_used_pages"] == stats["kv_kept_pages"]


def test_counters_and_the_per_step_profile_lines(monkeypatch, capfd):
    """stats() counts steps, tokens and the host's time by stage; with VIPERA_PROFILE_STEP=1 every
    step prints what it ran and the split of its device time by class of kernel, and every
    finished request a line in the shape of the reference's request log
    (crates/vipera-runtime/src/pipeline.rs:234-271, crates/vipera-backend-cpu/src/profile.rs:226-275)."""
    import json

    from vipera_rs_b200 import SamplingParams
    from vipera_rs_b200.kernels import ops

    vocab = helpers.CONFIGS["A"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 60 + n) for n in (20, 9)]
    folder, engine = _engine("A", "bfloat16", page_size=16, ctx=64, max_num_seqs=2, max_tokens_per_step=16)
    results = engine.generate(prompts, SamplingParams(max_new_tokens=5))
    stats = engine.stats()
    assert stats["steps"] >= 6 and stats["steps_with_portions"] >= 2
    assert stats["graph_steps"] == stats["steps"]            # every step replayed a captured graph
    assert stats["tokens_per_step"] * stats["steps"] == 29 + 2 * 4
    assert set(stats["host_micros_per_step"]) == {"allocate", "compute", "sample", "complete"}
    assert all(r.stage_micros["compute"] > 0 for r in results)
    monkeypatch.setenv("VIPERA_PROFILE_STEP", "1")
    try:
        _, profiled = _engine("A", "bfloat16", page_size=16, ctx=64, max_num_seqs=2, max_tokens_per_step=16)
        capfd.readouterr()
        again = profiled.generate(prompts, SamplingParams(max_new_tokens=5))
        lines = capfd.readouterr().err.splitlines()
    finally:
        ops.profile = None
    assert [r.tokens for r in again] == [r.tokens for r in results]
    steps = [line for line in lines if line.startswith("STEP ")]
    assert len(steps) == profiled.stats()["steps"] and all(" eager " in line for line in steps)
    assert any(" chunk " in line for line in steps) and any(" decode " in line for line in steps)
    split = [line for line in lines if line.startswith("PROFILE decode")]
    assert split and "proj" in split[-1] and "attention" in split[-1] and "norm" not in split[-1].split(":")[0]
    logs = [json.loads(line) for line in lines if line.startswith("{")]
    assert len(logs) == 2 and all(log["event"] == "generation" and log["finish"] == "length" for log in logs)
    assert {log["prompt_tokens"] for log in logs} == {20, 9}
    assert all(set(log["stage_micros"]) == {"allocate", "compute", "sample", "complete"} for log in logs)


def test_logprobs_of_the_drawn_tokens_and_the_most_likely_ones():
    """A request that asks for log-probabilities gets, for every generated token, its log-probability
    and the n most likely tokens with theirs, as the plain restatement of the reference's
    formula gives them on the plain logits; a request beside it that did not ask gets none, and
    its tokens are what it gets alone."""
    import plain_sampler
    from vipera_rs_b200 import SamplingParams

    folder, engine = _engine("A", "float32", page_size=16, ctx=128, max_num_seqs=3)
    vocab = helpers.CONFIGS["A"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 70 + n) for n in (11, 30, 6)]
    params = [SamplingParams(max_new_tokens=7, logprobs=4),
              SamplingParams(max_new_tokens=9),
              SamplingParams(max_new_tokens=6, temperature=0.7, seed=3, logprobs=0)]
    results = engine.generate(prompts, params)
    assert results[1].logprobs is None and results[1].top_logprobs is None
    assert results[1].tokens == engine.generate([prompts[1]], params[1])[0].tokens
    for prompt, asked, result in ((prompts[0], params[0], results[0]), (prompts[2], params[2], results[2])):
        assert len(result.logprobs) == len(result.tokens) == len(result.top_logprobs)
        logits = helpers.plain_logits(folder, list(prompt) + result.tokens[:-1])
        for index, token in enumerate(result.tokens):
            row = [plain_sampler.f32(float(v)) for v in logits[len(prompt) - 1 + index]]
            want, want_top = plain_sampler.logprobs(row, token, asked.temperature, asked.logprobs)
            assert abs(result.logprobs[index] - want) < 2e-4, (index, result.logprobs[index], want)
            got_top = result.top_logprobs[index]
            assert [i for i, _ in got_top] == [i for i, _ in want_top]
            assert all(abs(a - b) < 2e-4 for (_, a), (_, b) in zip(got_top, want_top))
        if asked.temperature == 0.0:   # the greedy token is the most likely one
            assert all(top[0][0] == token for top, token in zip(result.top_logprobs, result.tokens))
    assert engine.pools.audit() == ""

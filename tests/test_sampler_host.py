"""The native host sampler against the plain restatement of the reference's sampler, and the
reference's own unit list (crates/vipera-sampler/src/lib.rs:737-1004): greedy ties go to the
lowest id, top-k 1 is argmax, NaN is skipped, the same seed replays, two tokens at 3:1 are
drawn 75 % / 25 % of the time, invalid options are refused."""
import math

import numpy as np
import pytest

import plain_sampler
import vipera_rs_b200  # noqa: F401
from vipera_rs_b200 import errors
from vipera_rs_b200.sampling import HostSampler, Rng, SamplingParams, draw_greedy, draw_temperature


def test_generator_matches_the_formula():
    for seed in (0, 1, 7, 1234, 2**63 + 5):
        native, plain = Rng(seed), plain_sampler.Rng(seed)
        for _ in range(16):
            assert native.next_u64() == plain.next_u64()
        value = native.next_f64()
        assert value == plain.next_f64() and 0.0 <= value < 1.0
    assert Rng(1).next_u64() != Rng(2).next_u64()


def test_greedy():
    logits = np.array([0.5, 2.0, float("nan"), 2.0, float("inf"), -1.0], dtype=np.float32)
    assert draw_greedy(logits) == 1                    # NaN and inf skipped, the tie goes to the lower id
    assert draw_greedy(np.full(9, 0.25, dtype=np.float32)) == 0
    with pytest.raises(errors.InternalError):
        draw_greedy(np.array([float("nan"), float("-inf")], dtype=np.float32))


@pytest.mark.parametrize("seed", range(5))
def test_temperature_matches_the_plain_sampler(seed):
    rng = np.random.default_rng(seed)
    vocab = 3001
    logits = (rng.standard_normal(vocab) * 3).astype(np.float32)
    logits[17] = np.nan
    logits[100] = logits[200]                          # a tie inside the ranking
    uniform = plain_sampler.Rng(seed)
    for config in (dict(temperature=0.8, top_k=40, top_p=0.95, min_p=0.05),
                   dict(temperature=1.7, top_k=5, top_p=1.0, min_p=0.0),
                   dict(temperature=0.2, top_k=1, top_p=0.95, min_p=0.05),
                   dict(temperature=1.0, top_k=500, top_p=0.3, min_p=0.0),
                   dict(temperature=1.0, top_k=0, top_p=0.9, min_p=0.01)):
        for _ in range(20):
            u = uniform.next_f64()
            want = plain_sampler.temperature([float(x) for x in logits], config["temperature"], config["top_k"],
                                             config["top_p"], config["min_p"], u)
            assert draw_temperature(logits, config, [], u) == want, config
    assert draw_temperature(logits, dict(temperature=0.5, top_k=1, top_p=0.95, min_p=0.05), [], 0.999) == \
        plain_sampler.greedy([float(x) for x in logits])


def test_no_cut_reaches_past_the_bounded_head_when_the_mass_needs_it():
    """top_k = 0 and a flat distribution: the head of 4096 does not reach top_p, so every logit
    is ranked (crates/vipera-sampler/src/lib.rs:206-216)."""
    vocab = 6000
    logits = np.zeros(vocab, dtype=np.float32)
    config = dict(temperature=1.0, top_k=0, top_p=0.95, min_p=0.0)
    assert draw_temperature(logits, config, [], 0.9) == int(0.9 * 0.95 * vocab)


def test_penalties_match_the_plain_sampler():
    logits = np.array([2.0, -1.0, 0.5, 3.0, 1.0], dtype=np.float32)
    recent = [0, 0, 1, 4]
    config = dict(temperature=0.0, repetition_penalty=2.0, presence_penalty=0.5, frequency_penalty=0.25,
                  logit_bias=[(3, -100.0)])
    plain = plain_sampler.penalised([float(x) for x in logits], recent, 2.0, 0.5, 0.25, [(3, -100.0)])
    assert plain == pytest.approx([2.0 / 2 - 1.0, -2.0 - 0.75, 0.5, -97.0, 0.5 - 0.75])
    assert draw_greedy(logits, config, recent) == plain_sampler.greedy(plain) == 2


def test_distribution_and_seed_replay():
    logits = np.full(64, -30.0, dtype=np.float32)
    logits[5], logits[9] = math.log(3.0), 0.0
    params = SamplingParams(temperature=1.0, top_k=40, top_p=1.0, min_p=0.0, seed=3)
    sampler = HostSampler(params)
    draws = [sampler.sample(logits) for _ in range(4000)]
    assert abs(draws.count(5) / 4000 - 0.75) < 0.05 and set(draws) == {5, 9}
    again = HostSampler(params)
    assert [again.sample(logits) for _ in range(50)] == draws[:50]
    other = HostSampler(SamplingParams(temperature=1.0, top_k=40, top_p=1.0, min_p=0.0, seed=4))
    assert [other.sample(logits) for _ in range(50)] != draws[:50]
    greedy = HostSampler(SamplingParams(temperature=0.0))
    assert greedy.sample(logits) == 5


@pytest.mark.parametrize("bad", [dict(temperature=-0.1), dict(temperature=float("nan")), dict(top_p=0.0),
                                 dict(top_p=1.5), dict(min_p=1.0), dict(min_p=-0.1), dict(repetition_penalty=0.0),
                                 dict(presence_penalty=2.5), dict(frequency_penalty=-3.0),
                                 dict(logit_bias=[(1, 101.0)]), dict(logit_bias=[(i, 0.0) for i in range(17)])])
def test_invalid_options_are_refused(bad):
    with pytest.raises(errors.InvalidArgumentError):
        HostSampler(bad)

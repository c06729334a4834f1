"""The scheduler's decisions, driven by a toy step function (no GPU): the next token of a
request is a function of its last token and position, as in the reference's toy forward
passes (crates/vipera-runtime/src/engine.rs:1269-1331).  Invariants taken from the
reference's list (engine.rs:1490-1941, 2005-2142): a request's tokens do not depend on what
runs beside it or on arrival order; a long prompt does not starve decodes; a full cache ends
or postpones requests instead of failing them; cancel frees pages at once."""
import numpy as np
import pytest

import vipera_rs_b200  # noqa: F401
from vipera_rs_b200 import errors
from vipera_rs_b200.build import runtime_module

VOCAB = 97


def toy_token(tokens, position):
    return (tokens[position] * 7 + position * 3 + 1) % VOCAB


class ToyEngine:
    """Scheduler + cache manager + a step that needs no model."""

    def __init__(self, pages=64, page_size=16, max_num_seqs=4, budget=64, portion=64, window_group=False, reuse=False):
        rt = runtime_module()
        groups = [(page_size, pages, 0)] + ([(page_size, pages, 24)] if window_group else [])
        self.cache = rt.CacheManager(groups, max_num_seqs, reuse)
        self.scheduler = rt.Scheduler(self.cache, max_num_seqs, budget, portion, 0, reuse)
        self.history = {}       # request -> every token the step function has seen, by position
        self.prompts = {}
        self.cached = {}        # physical page -> the tokens whose keys the step function "wrote" there
        self.steps = []
        self.finished = {}

    def add(self, request, prompt, **params):
        params.setdefault("temperature", 0.0)
        self.prompts[request] = list(prompt)
        self.scheduler.add(request, list(prompt), params)

    def step(self):
        plan = self.scheduler.schedule()
        sampled = []
        if not plan.empty:
            tokens, positions = plan.tokens, plan.positions
            offset = 0
            for request, start, count, fresh in zip(plan.requests, plan.starts, plan.counts, plan.fresh):
                seen = self.history.setdefault(request, [])
                page = self.cache.group(0)[0]
                if fresh:
                    # what was not computed again must lie in the pages the request was given
                    assert start == 0 or self.cache.reuse
                    assert start % page == 0
                    del seen[:]
                    table = self.cache.table(request, 0)
                    for index in range(start // page):
                        seen.extend(self.cached[int(table[index])])
                    assert seen == (self.prompts[request] + self.finished.get(request, {}).get("tokens", []))[:start] \
                        or seen == self.known(request)[:start]
                assert len(seen) == start, "portions of a request must arrive in order, without gaps"
                assert positions[offset:offset + count].tolist() == list(range(start, start + count))
                seen.extend(tokens[offset:offset + count].tolist())
                table = self.cache.table(request, 0)
                for index in range(start // page, (start + count + page - 1) // page):
                    self.cached[int(table[index])] = seen[index * page:(index + 1) * page]
                # every position of the portion has its page
                table = self.cache.table(request, 0)
                assert all(table[p // self.cache.group(0)[0]] >= 0 for p in range(start, start + count))
                offset += count
            for request, index in zip(plan.row_requests, plan.row_token_index):
                seen = self.history[request]
                assert plan.positions[index] == len(seen) - 1, "logits are wanted at a request's last token"
                sampled.append(toy_token(seen, len(seen) - 1))
            self.steps.append((list(plan.requests), plan.counts.tolist(), list(plan.preempted)))
        outcome = self.scheduler.complete(plan, sampled)
        for item in outcome["finished"]:
            self.finished[item["request"]] = item
        assert self.cache.audit() == ""
        return plan, outcome

    def known(self, request):
        """The request's tokens so far as the test knows them: prompt, then what the toy step drew."""
        tokens = list(self.prompts[request])
        while len(tokens) < len(self.history.get(request, [])) + 64:
            tokens.append(toy_token(tokens, len(tokens) - 1))
        return tokens

    def run(self, limit=10000):
        for _ in range(limit):
            if not self.scheduler.has_work():
                return
            self.step()
        raise AssertionError("the scheduler did not finish")


def expected_tokens(prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(toy_token(tokens, len(tokens) - 1))
    return tokens[len(prompt):]


def test_one_request_prefills_in_portions_then_decodes():
    engine = ToyEngine(budget=48, portion=48)
    prompt = list(range(1, 101))
    engine.add(0, prompt, max_new_tokens=5)
    engine.run()
    counts = [c for _, cs, _ in engine.steps for c in cs]
    assert counts[:3] == [48, 48, 4] and counts[3:] == [1, 1, 1, 1]
    done = engine.finished[0]
    assert done["reason"] == "length" and done["tokens"] == expected_tokens(prompt, 5)
    assert done["prompt_tokens"] == 100 and done["processed_tokens"] == 104
    assert engine.cache.stats(0)["used_pages"] == 0 and engine.cache.open_requests() == []


def test_tokens_do_not_depend_on_company_or_arrival_order():
    prompts = {i: [(i * 13 + j) % VOCAB for j in range(n)] for i, n in enumerate([5, 100, 257, 31, 64])}
    alone = {}
    for request, prompt in prompts.items():
        engine = ToyEngine()
        engine.add(request, prompt, max_new_tokens=24)
        engine.run()
        alone[request] = engine.finished[request]["tokens"]
        assert alone[request] == expected_tokens(prompt, 24)
    for order in ([0, 1, 2, 3, 4], [4, 2, 0, 3, 1]):
        engine = ToyEngine(max_num_seqs=3, budget=48, portion=48)
        for request in order:
            engine.add(request, prompts[request], max_new_tokens=24)
        engine.run()
        for request in prompts:
            assert engine.finished[request]["tokens"] == alone[request]
        # portions of prompts ran beside decode tokens in the same steps
        assert any(len(cs) > 1 and 1 in cs and max(cs) > 1 for _, cs, _ in engine.steps)
        assert all(sum(cs) <= 48 for _, cs, _ in engine.steps)


def test_a_long_prompt_does_not_starve_a_decoding_request():
    engine = ToyEngine(budget=32, portion=32, pages=128)
    engine.add(0, [1, 2, 3], max_new_tokens=40)
    engine.step()
    engine.add(1, list(range(600)), max_new_tokens=2)
    while 1 not in engine.finished:
        plan, _ = engine.step()
        if 0 not in engine.finished:
            assert 0 in plan.requests, "the decoding request takes part in every step"
    engine.run()
    assert engine.finished[0]["tokens"] == expected_tokens([1, 2, 3], 40)


def test_stop_token_and_limits():
    prompt = [5, 6, 7]
    tokens = expected_tokens(prompt, 10)
    engine = ToyEngine()
    engine.add(0, prompt, max_new_tokens=10, eos_ids=[tokens[3]])
    engine.run()
    assert engine.finished[0]["reason"] == "stop" and engine.finished[0]["tokens"] == tokens[:4]
    rt = runtime_module()
    cache = rt.CacheManager([(16, 8, 0)], 2)
    scheduler = rt.Scheduler(cache, 2, 64, 64, 20)             # max_model_len 20
    scheduler.add(0, list(range(15)), {"max_new_tokens": 50, "temperature": 0.0})
    finished = None
    for _ in range(50):
        plan = scheduler.schedule()
        outcome = scheduler.complete(plan, [1] * plan.num_rows)
        if outcome["finished"]:
            finished = outcome["finished"][0]
            break
    assert finished["reason"] == "length" and len(finished["tokens"]) == 5


def test_admission_refusals():
    engine = ToyEngine(pages=4)                                # 64 tokens of cache
    with pytest.raises(errors.InvalidArgumentError):
        engine.add(0, [], max_new_tokens=1)
    with pytest.raises(errors.InvalidArgumentError):
        engine.add(0, [1], max_new_tokens=0)
    with pytest.raises(errors.InfeasibleError):
        engine.add(0, list(range(64)), max_new_tokens=1)       # the prompt alone fills the cache
    with pytest.raises(errors.InvalidArgumentError):
        engine.add(0, [1], max_new_tokens=1, temperature=-1.0)
    engine.add(0, [1], max_new_tokens=1)
    with pytest.raises(errors.InvalidArgumentError):
        engine.add(0, [2], max_new_tokens=1)                   # the id is in use


def test_when_pages_run_out_the_last_admitted_starts_over():
    """Four requests, pages for about two and a half: the one admitted last gives its pages
    back, waits at the head of the line, and is computed again; every request still ends with
    the tokens it gets alone, and nothing is reported as an error."""
    engine = ToyEngine(pages=14, budget=64, portion=64)
    prompts = {i: [(i + j * 5) % VOCAB for j in range(n)] for i, n in enumerate([40, 50, 60, 30])}
    for request, prompt in prompts.items():
        engine.add(request, prompt, max_new_tokens=40)
    engine.run()
    preempted = [r for _, _, ps in engine.steps for r in ps]
    assert preempted, "the cache was made too small for all four"
    for request, prompt in prompts.items():
        done = engine.finished[request]
        assert done["reason"] == "length" and done["tokens"] == expected_tokens(prompt, 40)
    assert sum(engine.finished[r]["preemptions"] for r in prompts) == len(preempted)
    victim = preempted[0]
    assert engine.finished[victim]["processed_tokens"] > len(prompts[victim]) + 40   # it was recomputed
    assert engine.cache.stats(0)["used_pages"] == 0


def test_a_request_alone_that_cannot_grow_ends_with_length():
    engine = ToyEngine(pages=3, page_size=16)                  # 48 tokens at most
    engine.add(0, list(range(40)), max_new_tokens=100)
    engine.run()
    done = engine.finished[0]
    # positions 0..47 fit: the prompt's last position gives token 1, position 47 gives token 9,
    # which no page is left to feed back
    assert done["reason"] == "length" and len(done["tokens"]) == 9
    assert engine.cache.stats(0)["used_pages"] == 0


def test_cancel_frees_pages_at_once():
    engine = ToyEngine()
    engine.add(0, list(range(50)), max_new_tokens=100)
    engine.add(1, list(range(20)), max_new_tokens=100)
    engine.step()
    engine.step()
    used = engine.cache.stats(0)["used_pages"]
    engine.scheduler.cancel(0)
    assert engine.cache.stats(0)["used_pages"] < used and not engine.cache.is_open(0)
    plan, outcome = engine.step()
    assert [f["reason"] for f in outcome["finished"] if f["request"] == 0] == ["cancelled"]
    assert plan.requests == [1]
    engine.scheduler.cancel(1)
    engine.run()
    assert engine.cache.stats(0)["used_pages"] == 0


def test_a_failed_step_ends_only_its_requests():
    engine = ToyEngine(max_num_seqs=2)
    engine.add(0, [1, 2, 3], max_new_tokens=5)
    engine.add(1, [4, 5, 6], max_new_tokens=5)
    engine.add(2, [7, 8, 9], max_new_tokens=5)                # waits: two run at once
    plan = engine.scheduler.schedule()
    outcome = engine.scheduler.fail(plan)
    assert sorted(f["request"] for f in outcome["finished"]) == [0, 1]
    assert all(f["reason"] == "error" for f in outcome["finished"])
    assert engine.cache.stats(0)["used_pages"] == 0
    engine.run()
    assert engine.finished[2]["tokens"] == expected_tokens([7, 8, 9], 5)


def test_sampling_rows_carry_each_requests_own_generator():
    rt = runtime_module()
    draws = []
    for company in (False, True):
        cache = rt.CacheManager([(16, 32, 0)], 4)
        scheduler = rt.Scheduler(cache, 4, 64, 64, 0)
        scheduler.add(0, [1, 2, 3], {"max_new_tokens": 4, "temperature": 0.8, "seed": 1234})
        if company:
            scheduler.add(1, [9, 9], {"max_new_tokens": 4, "temperature": 0.5, "seed": 99, "top_k": 7})
        mine = []
        for _ in range(4):
            plan = scheduler.schedule()
            index = plan.row_requests.index(0)
            mine.append(float(plan.row_uniform[index]))
            assert abs(float(plan.row_temperature[index]) - 0.8) < 1e-6 and int(plan.row_top_k[index]) == 40
            scheduler.complete(plan, [5] * plan.num_rows)
        draws.append(mine)
    assert draws[0] == draws[1]                                # the same numbers whatever runs beside it
    reference = rt.Rng(1234)
    assert draws[0] == [reference.next_f64() for _ in range(4)]


def test_penalty_rows_list_recent_tokens_with_counts():
    rt = runtime_module()
    cache = rt.CacheManager([(16, 32, 0)], 2)
    scheduler = rt.Scheduler(cache, 2, 64, 64, 0)
    scheduler.add(0, [4, 9, 4, 4, 7], {"max_new_tokens": 2, "temperature": 0.0, "repetition_penalty": 1.3,
                                       "frequency_penalty": 0.5, "logit_bias": [(11, -100.0)], "recent_window": 4})
    plan = scheduler.schedule()
    assert plan.any_penalty
    ids, counts, repetition, presence, frequency, bias = plan.row_penalty(0)
    assert ids.tolist() == [4, 7, 9] and counts.tolist() == [2, 1, 1]          # the last four tokens
    assert abs(repetition - 1.3) < 1e-6 and presence == 0.0 and frequency == 0.5
    assert bias == [(11, -100.0)]


def test_windowed_group_keeps_the_scheduler_going_past_its_pages():
    """With a windowed group the request holds only the window's pages there, so a long request
    fits although the group is small."""
    rt = runtime_module()
    cache = rt.CacheManager([(16, 40, 0), (16, 5, 24)], 2)
    scheduler = rt.Scheduler(cache, 2, 32, 32, 0)
    scheduler.add(0, list(range(200)), {"max_new_tokens": 100, "temperature": 0.0})
    produced = 0
    for _ in range(400):
        if not scheduler.has_work():
            break
        plan = scheduler.schedule()
        outcome = scheduler.complete(plan, [3] * plan.num_rows)
        produced += len(outcome["tokens"])
        assert cache.audit() == "" and cache.stats(1)["used_pages"] <= 5
    assert produced == 100


def test_a_prompt_seen_before_is_not_computed_again():
    """Prefix reuse (the reference: crates/vipera-runtime/src/engine.rs:432-491 and its tests
    :2005-2110): whole pages of a prompt an earlier request computed are taken over, at least
    one token is always computed, the tokens drawn are the same, and the pages are given up
    when others need them."""
    engine = ToyEngine(pages=12, page_size=8, max_num_seqs=2, budget=64, portion=64, reuse=True)
    prompt = [(i * 5 + 2) % VOCAB for i in range(37)]
    engine.add(1, prompt, max_new_tokens=6)
    engine.run()
    first = engine.finished[1]
    assert first["reused_tokens"] == 0 and first["processed_tokens"] == 37 + 5
    assert engine.cache.stats(0)["kept_pages"] == 4          # 37 tokens: four full pages of the prompt stay
    engine.add(2, prompt, max_new_tokens=6)
    engine.add(3, prompt[:20] + [1, 2, 3], max_new_tokens=4)
    engine.run()
    again, branch = engine.finished[2], engine.finished[3]
    assert again["tokens"] == first["tokens"] == expected_tokens(prompt, 6)
    assert again["reused_tokens"] == 32 and again["processed_tokens"] == 5 + 5
    assert branch["reused_tokens"] == 16 and branch["tokens"] == expected_tokens(prompt[:20] + [1, 2, 3], 4)
    # the whole prompt is known, one token is computed all the same
    engine.add(4, prompt[:32], max_new_tokens=2)
    engine.run()
    assert engine.finished[4]["reused_tokens"] == 24 and engine.finished[4]["tokens"] == expected_tokens(prompt[:32], 2)
    # requests with other prompts need the pages: the kept ones go, nobody is refused
    for request in range(10, 16):
        engine.add(request, [(request * 11 + i) % VOCAB for i in range(40)], max_new_tokens=8)
    engine.run()
    assert all(engine.finished[r]["reason"] == "length" for r in range(10, 16))
    assert engine.cache.audit() == ""


def test_a_request_put_back_finds_its_own_pages_again():
    """Preemption by recomputation costs little when prefixes are shared: the request put back
    published its prompt's pages, and takes them over when it is admitted again."""
    engine = ToyEngine(pages=7, page_size=8, max_num_seqs=2, budget=64, portion=64, reuse=True)
    engine.add(1, [(i * 3) % VOCAB for i in range(20)], max_new_tokens=30)
    engine.add(2, [(i * 7 + 1) % VOCAB for i in range(20)], max_new_tokens=12)
    engine.run()
    assert engine.finished[1]["tokens"] == expected_tokens([(i * 3) % VOCAB for i in range(20)], 30)
    assert engine.finished[2]["tokens"] == expected_tokens([(i * 7 + 1) % VOCAB for i in range(20)], 12)
    put_back = [item for item in engine.finished.values() if item["preemptions"] >= 1]
    assert put_back and all(item["reused_tokens"] >= 16 for item in put_back)


def test_the_step_after_is_foreseen_only_where_nothing_can_change_it():
    """plan_ahead(): true in a step where every running request decodes greedily and cannot end
    but by an end token; the pages for the token after are then reserved, and the next
    schedule() returns the same requests one position further.  False with a request waiting,
    a prompt portion in the step, a temperature, a penalty, or a request at its last token."""
    engine = ToyEngine(pages=32, max_num_seqs=2, budget=64, portion=64)
    engine.add(1, [3, 4, 5, 6, 7], max_new_tokens=6)
    engine.add(2, list(range(10, 27)), max_new_tokens=40)
    plan = engine.scheduler.schedule()
    assert not engine.scheduler.plan_ahead(plan)             # prompt portions
    engine.scheduler.complete(plan, [11, 12])
    foreseen = 0
    for step in range(12):
        plan = engine.scheduler.schedule()
        if plan.empty:
            break
        ahead = engine.scheduler.plan_ahead(plan)
        starts, requests = plan.starts.copy(), list(plan.requests)
        if ahead:
            foreseen += 1
            for request, start in zip(requests, starts):      # the page of the token after is there
                assert engine.cache.table(request, 0)[(start + 1) // 16] >= 0
        outcome = engine.scheduler.complete(plan, [20 + step] * plan.num_rows)
        assert engine.cache.audit() == ""
        following = engine.scheduler.schedule()
        if ahead:
            assert not outcome["finished"]
            assert list(following.requests) == requests and (following.starts == starts + 1).all()
            assert (following.counts == 1).all() and following.all_greedy
        # undo nothing: the plan just made is simply completed in the next round
        outcome = engine.scheduler.complete(following, [50 + step] * following.num_rows)
        assert engine.cache.audit() == ""
    assert foreseen >= 1

    # a request at its last token by the limit is not foreseen; one waiting blocks it too
    engine = ToyEngine(pages=32, max_num_seqs=1, budget=64, portion=64)
    engine.add(1, [3, 4, 5], max_new_tokens=2)
    engine.add(2, [9, 9], max_new_tokens=8)
    plan = engine.scheduler.schedule()
    engine.scheduler.complete(plan, [7])                       # first token of request 1; request 2 waits
    plan = engine.scheduler.schedule()
    assert not engine.scheduler.plan_ahead(plan)               # request 2 waits, and request 1 ends with this token
    outcome = engine.scheduler.complete(plan, [8])
    assert [item["request"] for item in outcome["finished"]] == [1]
    plan = engine.scheduler.schedule()                         # request 2's prompt
    engine.scheduler.complete(plan, [5])
    plan = engine.scheduler.schedule()
    assert engine.scheduler.plan_ahead(plan)                   # alone, greedy, 7 tokens to go
    engine.scheduler.complete(plan, [6])

    for params in ({"temperature": 0.8}, {"temperature": 0.0, "repetition_penalty": 1.3}):
        engine = ToyEngine(pages=32, max_num_seqs=1)
        engine.add(1, [3, 4, 5], max_new_tokens=8, **params)
        engine.scheduler.complete(engine.scheduler.schedule(), [7])
        plan = engine.scheduler.schedule()
        assert not engine.scheduler.plan_ahead(plan)
        engine.scheduler.complete(plan, [7])


def test_a_request_that_ends_after_its_next_step_was_foreseen_gives_every_page_back():
    engine = ToyEngine(pages=8, page_size=4, max_num_seqs=2)
    engine.add(1, [3, 4, 5, 6], max_new_tokens=20, eos_ids=[42])
    engine.scheduler.complete(engine.scheduler.schedule(), [7])
    plan = engine.scheduler.schedule()
    assert engine.scheduler.plan_ahead(plan)
    used = engine.cache.stats(0)["used_pages"]
    assert used == 2                                           # positions 0..5: the token after has its page
    outcome = engine.scheduler.complete(plan, [42])            # the end token, drawn while the step after ran
    assert [item["reason"] for item in outcome["finished"]] == ["stop"]
    assert engine.cache.stats(0)["used_pages"] == engine.cache.stats(0)["kept_pages"]
    assert engine.cache.audit() == ""
    assert not engine.scheduler.has_work()


def test_rows_with_a_temperature_are_foreseen_with_their_next_draws():
    """With a top-k the device sampler draws alone, a temperature does not stop plan_ahead();
    peek_uniforms() gives the draws the next schedule() hands out, without taking them."""
    engine = ToyEngine(pages=32, max_num_seqs=2)
    engine.add(1, [3, 4, 5], max_new_tokens=12, temperature=0.8, top_k=40, seed=7)
    engine.add(2, [6, 7], max_new_tokens=12, temperature=0.0)
    engine.scheduler.complete(engine.scheduler.schedule(), [9, 9])
    for step in range(4):
        plan = engine.scheduler.schedule()
        assert not engine.scheduler.plan_ahead(plan)            # greedy rows only, by default
        assert engine.scheduler.plan_ahead(plan, 4096)
        assert not engine.scheduler.plan_ahead(plan, 39)        # a top-k above what the caller's sampler takes
        peeked = engine.scheduler.peek_uniforms(plan)
        assert peeked[1] == 0.0 and 0.0 <= peeked[0] < 1.0
        assert np.array_equal(peeked, engine.scheduler.peek_uniforms(plan))   # looking takes nothing
        engine.scheduler.complete(plan, [10 + step, 20 + step])
        following = engine.scheduler.schedule()
        assert np.array_equal(following.row_uniform, peeked)
        engine.scheduler.complete(following, [30 + step, 40 + step])
    # without a top-k the whole vocabulary may be needed on the host: not foreseen
    engine = ToyEngine(pages=32, max_num_seqs=1)
    engine.add(1, [3, 4, 5], max_new_tokens=8, temperature=0.8, top_k=0)
    engine.scheduler.complete(engine.scheduler.schedule(), [7])
    assert not engine.scheduler.plan_ahead(engine.scheduler.schedule(), 4096)

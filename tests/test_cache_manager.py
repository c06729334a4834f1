"""The cache manager's books: pages and state slots under ordinary use and under random
orders of requests.  Unit cases follow the reference's list (crates/vipera-runtime/src/kv.rs:572-901):
block arithmetic, lowest page first, a failed reservation leaves nothing behind, release
returns everything; windows and groups are this engine's additions."""
import random

import numpy as np
import pytest

import vipera_rs_b200  # noqa: F401
from vipera_rs_b200 import errors
from vipera_rs_b200.build import runtime_module


def manager(groups, slots=4, reuse=False):
    return runtime_module().CacheManager(groups, slots, reuse)


def test_pages_are_handed_out_lowest_first_and_counted():
    cache = manager([(16, 8, 0)])
    assert cache.open(7) == 0
    cache.reserve(7, 33)                      # 33 tokens need 3 pages of 16
    assert cache.table(7, 0).tolist() == [0, 1, 2]
    assert cache.stats(0) == {"total_pages": 8, "free_pages": 5, "used_pages": 3, "kept_pages": 0}
    cache.reserve(7, 48)                      # still 3 pages
    assert cache.table(7, 0).tolist() == [0, 1, 2]
    cache.commit(7, 48)
    assert cache.computed(7) == 48
    cache.open(9)
    cache.reserve(9, 1)
    assert cache.table(9, 0).tolist() == [3]
    cache.close(7)
    assert cache.stats(0)["free_pages"] == 7
    cache.open(11)
    cache.reserve(11, 17)
    assert cache.table(11, 0).tolist() == [0, 1]   # the lowest page of the released request comes first
    assert cache.audit() == ""


def test_a_failed_reservation_leaves_nothing_behind():
    cache = manager([(16, 4, 0), (16, 2, 0)])      # the second group is the tighter one
    cache.open(1)
    cache.reserve(1, 20)
    before = (cache.table(1, 0).tolist(), cache.table(1, 1).tolist(), cache.stats(0), cache.stats(1))
    assert not cache.fits(1, 40)
    with pytest.raises(errors.InfeasibleError):
        cache.reserve(1, 40)                       # group 0 could, group 1 cannot: nothing is taken
    assert (cache.table(1, 0).tolist(), cache.table(1, 1).tolist(), cache.stats(0), cache.stats(1)) == before
    assert cache.longest_fit(1, 1000) == 32
    assert cache.audit() == ""


def test_state_slots_and_errors():
    cache = manager([(16, 4, 0)], slots=2)
    assert cache.open(1) == 0 and cache.open(2) == 1
    with pytest.raises(errors.InfeasibleError):
        cache.open(3)
    with pytest.raises(errors.InvalidArgumentError):
        cache.open(1)
    cache.close(1)
    assert cache.open(3) == 0                      # the slot is used again
    with pytest.raises(errors.InvalidArgumentError):
        cache.close(99)
    with pytest.raises(errors.InvalidArgumentError):
        cache.commit(2, 5)                         # nothing was reserved for these tokens
    with pytest.raises(errors.InvalidArgumentError):
        manager([(0, 4, 0)])
    assert cache.capacity_tokens() == 64 and cache.could_ever_fit(64) and not cache.could_ever_fit(65)


def test_a_window_gives_pages_back_as_it_passes_them():
    cache = manager([(16, 100, 0), (16, 6, 40)])   # group 1: a window of 40 keys
    cache.open(1)
    done = 0
    held = []
    while done < 400:
        step = 23
        cache.reserve(1, done + step)
        cache.commit(1, done + step)
        done += step
        table = cache.table(1, 1)
        live = [i for i, page in enumerate(table.tolist()) if page >= 0]
        held.append(len(live))
        # every key the next query can read has its page: positions done-39 .. done-1
        first_needed = max(0, done - 40 + 1) // 16
        assert live and live[0] <= first_needed and live[-1] == (done - 1) // 16
        assert all(table[i] >= 0 for i in range(first_needed, (done - 1) // 16 + 1))
        assert cache.audit() == ""
    assert max(held) <= 5                          # window + one portion, never the whole history
    assert cache.stats(0)["used_pages"] == (done + 15) // 16
    cache.close(1)
    assert cache.stats(1)["free_pages"] == 6 and cache.stats(0)["free_pages"] == 100


def test_tables_for_a_step():
    cache = manager([(16, 16, 0)])
    for request, length in ((5, 40), (6, 3)):
        cache.open(request)
        cache.reserve(request, length)
    tables = cache.tables([6, 5], 0, 4)
    assert tables.dtype == np.int32 and tables.shape == (2, 4)
    assert tables.tolist() == [[3, -1, -1, -1], [0, 1, 2, -1]]
    with pytest.raises(errors.InvalidArgumentError):
        cache.tables([5], 0, 2)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_duplicate_a_page(seed):
    rng = random.Random(seed)
    groups = [(16, 24, 0), (8, 20, 24)] if seed % 2 else [(32, 12, 0)]
    cache = manager(groups, slots=5)
    live = {}
    next_id = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            cache.open(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.75 and live:
            request = rng.choice(list(live))
            grow = rng.randint(1, 70)
            target = live[request] + grow
            if cache.fits(request, target):
                cache.reserve(request, target)
                if rng.random() < 0.9:
                    cache.commit(request, target)
                    live[request] = target
            else:
                with pytest.raises(errors.InfeasibleError):
                    cache.reserve(request, target)
                shorter = cache.longest_fit(request, target)
                assert live[request] <= shorter < target
                cache.reserve(request, shorter)
                cache.commit(request, shorter)
                live[request] = shorter
        elif live:
            request = rng.choice(list(live))
            cache.close(request)
            del live[request]
        assert cache.audit() == "", cache.audit()
        for g in range(cache.num_groups):
            stats = cache.stats(g)
            held = sum(int((cache.table(r, g) >= 0).sum()) for r in live)
            assert stats["used_pages"] == held and stats["free_pages"] + held == stats["total_pages"]
        assert cache.free_state_slots == 5 - len(live)
    for request in list(live):
        cache.close(request)
        with pytest.raises(errors.InvalidArgumentError):
            cache.close(request)                   # a second release is refused, not repeated
    assert cache.audit() == ""
    assert all(cache.stats(g)["free_pages"] == groups[g][1] for g in range(len(groups)))


def test_published_pages_are_shared_not_copied_and_given_up_when_pages_are_needed():
    """The reference parks a finished sequence's blocks, copies a matching prefix and evicts
    parked blocks oldest first when the free list runs dry (crates/vipera-runtime/src/kv.rs:
    427-514, tests :730-901).  Here the pages themselves are shared."""
    cache = manager([(4, 8, 0)], slots=3, reuse=True)
    assert cache.reuse
    prompt = list(range(100, 114))                       # 14 tokens: three full pages and a rest
    cache.open(1)
    assert cache.match(1, prompt) == 0                   # nothing is known yet
    cache.reserve(1, 14)
    cache.commit(1, 14)
    cache.publish(1, prompt, 14)
    assert cache.table(1, 0).tolist() == [0, 1, 2, 3]
    cache.open(2)                                        # same beginning, then something else
    other = prompt[:9] + [7, 7, 7]
    assert cache.match(2, other) == 8                    # two full pages agree
    assert cache.table(2, 0).tolist() == [0, 1] and cache.computed(2) == 8
    cache.reserve(2, 12)
    assert cache.table(2, 0).tolist() == [0, 1, 4]       # its own page from the free stack
    assert cache.audit() == ""
    cache.close(1)
    assert cache.stats(0) == {"total_pages": 8, "free_pages": 4, "used_pages": 4, "kept_pages": 1}
    cache.open(3)                                        # the whole prompt again: one token must stay to compute
    assert cache.match(3, prompt[:13]) == 12
    cache.close(3)
    cache.close(2)
    assert cache.stats(0)["kept_pages"] == 3 and cache.stats(0)["free_pages"] == 5
    # a request that needs every page gets them: the published ones are given up, deepest first
    cache.open(4)
    assert cache.fits(4, 32) and not cache.fits(4, 33)
    cache.reserve(4, 30)
    assert cache.stats(0)["kept_pages"] == 0 and cache.audit() == ""
    cache.close(4)
    cache.open(5)
    assert cache.match(5, prompt) == 0                   # given up means forgotten
    cache.close(5)
    assert cache.stats(0)["free_pages"] == 8 and cache.audit() == ""


def test_no_sharing_with_windows_or_unequal_pages():
    assert not manager([(16, 8, 0), (16, 8, 24)], reuse=True).reuse
    assert not manager([(16, 8, 0), (8, 8, 0)], reuse=True).reuse
    assert manager([(16, 8, 0), (16, 4, 0)], reuse=True).reuse
    assert not manager([(16, 8, 0)], reuse=False).reuse


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_with_shared_prefixes(seed):
    """Requests drawn from a few prompts with common beginnings come, grow, publish and go in
    random order, in a pool so small that published pages are given up all the time.  After
    every action the books are sound, and a page a request was given by a match holds what
    that request's own tokens say (the test keeps, for every page, the tokens whose keys were
    written to it)."""
    rng = random.Random(seed)
    page = 4
    cache = manager([(page, 14, 0), (page, 14, 0)], slots=4, reuse=True)
    stems = [[rng.randrange(50) for _ in range(40)] for _ in range(3)]
    written = {}                                         # physical page -> (first position, tokens)
    live = {}
    next_id = 0

    def check_tables(request):
        tokens, done = live[request]
        table = cache.table(request, 0)
        assert len(cache.table(request, 1)) == len(table)
        for index in range(done // page):
            first, content = written[int(table[index])]
            assert first == index * page and content == tokens[index * page:(index + 1) * page], (request, index)

    for _ in range(500):
        action = rng.random()
        if action < 0.3 and len(live) < 4:
            stem = rng.choice(stems)
            cut = rng.randint(2, 40)
            tokens = stem[:cut] + [rng.randrange(50) for _ in range(rng.randint(0, 12))]
            cache.open(next_id)
            reused = cache.match(next_id, tokens)
            assert reused % page == 0 and reused < len(tokens) and reused == cache.computed(next_id)
            live[next_id] = (tokens, reused)
            check_tables(next_id)
            next_id += 1
        elif action < 0.75 and live:
            request = rng.choice(list(live))
            tokens, done = live[request]
            if done == len(tokens):
                continue
            target = min(len(tokens), done + rng.randint(1, 9))
            target = cache.longest_fit(request, target)
            if target == done:
                continue
            cache.reserve(request, target)
            table = cache.table(request, 0)
            for index in range(done // page, (target + page - 1) // page):     # pages this portion writes
                written[int(table[index])] = (index * page, list(tokens[index * page:min(target, (index + 1) * page)]))
            cache.commit(request, target)
            live[request] = (tokens, target)
            cache.publish(request, tokens, target)
            check_tables(request)
        elif live:
            request = rng.choice(list(live))
            cache.close(request)
            del live[request]
        assert cache.audit() == "", cache.audit()
        stats = cache.stats(0)
        distinct = {int(p) for r in live for p in cache.table(r, 0) if p >= 0}
        assert stats["used_pages"] == len(distinct) + stats["kept_pages"]
    for request in list(live):
        cache.close(request)
    assert cache.audit() == ""


def test_decode_step_inputs_are_filled_in_the_graphs_layout():
    """The native routine behind the decode graphs: tokens, positions, state slots, fresh marks
    and block tables of the step's requests in one buffer, entries past the step's own
    repeating its first; -1 for a step that is not a plain decode step; errors for a token
    outside the vocabulary, a position past the limit, and a position without a page."""
    cache = manager([(16, 8, 0), (8, 8, 0)], slots=4)
    for request, length in ((5, 20), (9, 3)):
        cache.open(request)
        cache.reserve(request, length)
    bucket, widths = 4, [2, 4]
    total = 8 * bucket + 1 + bucket * sum(widths)
    buffer = np.full(total, -7, dtype=np.int32)

    def fill(tokens, counts, pos0, fresh, rows, requests=(5, 9), vocab=100, limit=64):
        return cache.fill_decode(list(requests), np.asarray(tokens, dtype=np.int32), counts, pos0, fresh, rows,
                                 buffer.ctypes.data, bucket, widths, vocab, limit)

    assert fill([11, 22], [1, 1], [19, 2], [0, 1], [0, 1]) == 2
    b = bucket
    assert buffer[:b].tolist() == [11, 22, 11, 11]                      # tokens
    assert buffer[b:2 * b].tolist() == [19, 2, 19, 19]                  # positions
    assert buffer[2 * b:4 * b + 1].tolist() == [-7] * (2 * b + 1)       # the caller's constant parts
    assert buffer[4 * b + 1:5 * b + 1].tolist() == [19, 2, 19, 19]      # first positions
    assert buffer[5 * b + 1:6 * b + 1].tolist() == [0, 1, 0, 0]         # state slots
    assert buffer[6 * b + 1:7 * b + 1].tolist() == [0, 1, 0, 0]         # fresh
    assert buffer[7 * b + 1:8 * b + 1].tolist() == [-7] * b
    first = buffer[8 * b + 1:8 * b + 1 + b * 2].reshape(b, 2)
    assert first.tolist() == [cache.table(5, 0).tolist(), cache.table(9, 0).tolist() + [-1]] + [cache.table(5, 0).tolist()] * 2
    second = buffer[8 * b + 1 + b * 2:].reshape(b, 4)
    assert second[0].tolist() == cache.table(5, 1).tolist() + [-1] and second[1].tolist() == cache.table(9, 1).tolist() + [-1] * 3
    assert second[2].tolist() == second[0].tolist()
    # not a plain decode step: a portion of two tokens, rows in another order, fewer rows than entries
    assert fill([1, 2, 3], [2, 1], [18, 2], [0, 0], [0, 1]) == -1
    assert fill([1, 2], [1, 1], [19, 2], [0, 0], [1, 0]) == -1
    assert fill([1, 2], [1, 1], [19, 2], [0, 0], [0]) == -1
    with pytest.raises(errors.InvalidArgumentError):
        fill([1, 100], [1, 1], [19, 2], [0, 0], [0, 1])                 # token outside the vocabulary
    with pytest.raises(errors.InvalidArgumentError):
        fill([1, 2], [1, 1], [19, 2], [0, 0], [0, 1], limit=19)         # position past the limit
    with pytest.raises(errors.InvalidArgumentError):
        fill([1, 2], [1, 1], [19, 9], [0, 0], [0, 1])                   # request 9 has no page of 8 keys for position 9

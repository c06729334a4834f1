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


def manager(groups, slots=4):
    return runtime_module().CacheManager(groups, slots)


def test_pages_are_handed_out_lowest_first_and_counted():
    cache = manager([(16, 8, 0)])
    assert cache.open(7) == 0
    cache.reserve(7, 33)                      # 33 tokens need 3 pages of 16
    assert cache.table(7, 0).tolist() == [0, 1, 2]
    assert cache.stats(0) == {"total_pages": 8, "free_pages": 5, "used_pages": 3}
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

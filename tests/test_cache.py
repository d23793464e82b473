"""The cache manager on the host: no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; state slots (no GPU)."""
import random

import pytest

from tokenizer_b200.cache import (CachePlan, OutOfPages, PageAllocator, PageError, pages_for,
                                  prefix_hash)
from tokenizer_b200.parts.base import CacheNeed, KVNeed, StateNeed


def test_stack_order_and_round_trip():
    a = PageAllocator(4, 16)
    assert [a.take() for _ in range(4)] == [0, 1, 2, 3]     # first page handed out is 0
    assert a.take() is None and a.available == 0
    assert a.give_back(2) == "freed" and a.give_back(0) == "freed"
    assert a.take() == 0 and a.take() == 2                   # last freed, first reused
    a.check()


def test_double_free_and_unknown():
    a = PageAllocator(2, 16)
    p = a.take()
    a.give_back(p)
    with pytest.raises(PageError, match="double free"):
        a.give_back(p)
    with pytest.raises(PageError, match="not issued"):
        a.give_back(7)
    with pytest.raises(PageError, match="cannot gain a holder"):
        a.hold(p)


def test_take_n_is_all_or_nothing():
    a = PageAllocator(3, 16)
    assert a.take_n(4) is None and a.free_count == 3
    assert sorted(a.take_n(3)) == [0, 1, 2]
    assert a.take_n(1) is None


def test_hash_chain_matches_the_formula():
    value = 0xCBF29CE484222325
    for t in (5, 70000):
        value = ((value ^ t) * 0x100000001B3) & ((1 << 64) - 1)
    assert prefix_hash(0, [5, 70000]) == value
    assert prefix_hash(3, [5]) != prefix_hash(4, [5])


def test_prefix_sharing_and_eviction():
    a = PageAllocator(4, 4)
    prompt = list(range(10))                       # two full pages and a tail
    pages = a.take_n(3)
    a.publish_prompt(prompt, pages)
    shared = a.take_shared_prefix(prompt[:9])
    assert shared == pages[:2] and a.holders(pages[0]) == 2
    # a prompt that differs inside the second page shares only the first
    other = prompt[:5] + [99] + prompt[6:]
    assert a.take_shared_prefix(other) == pages[:1]
    for p in shared + pages[:1]:
        assert a.give_back(p) == "shared"
    assert [a.give_back(p) for p in pages] == ["kept", "kept", "freed"]
    assert a.kept_count == 2 and a.available == 4
    # kept pages are found again, and are evicted (oldest first) only when the stack is empty
    again = a.take_shared_prefix(prompt)
    assert again == pages[:2]
    for p in again:
        a.give_back(p)
    taken = a.take_n(4)
    assert taken is not None and a.kept_count == 0
    assert a.take_shared_prefix(prompt) == []      # evicted pages are forgotten
    a.check()


def test_colliding_hash_never_shares(monkeypatch):
    import tokenizer_b200.cache.allocator as mod
    monkeypatch.setattr(mod, "prefix_hash", lambda parent, tokens: 42)
    a = PageAllocator(4, 2)
    p = a.take_n(1)
    a.publish_prompt([1, 2], p)
    assert a.take_shared_prefix([3, 4]) == []      # same hash, other ids
    assert a.take_shared_prefix([1, 2]) == p


def needs(n_full, n_window=0, window=None, state=False):
    out = [CacheNeed(kv=KVNeed(2, 16, None)) for _ in range(n_full)]
    out += [CacheNeed(kv=KVNeed(2, 16, window)) for _ in range(n_window)]
    if state:
        out.append(CacheNeed(state=StateNeed((4,))))
    return out


def test_groups_follow_what_mixers_store():
    plan = CachePlan(needs(2, 2, window=8, state=True) + [None], 8, 4, 3)
    assert [(g.window, g.calls) for g in plan.groups] == [(None, [0, 1]), (8, [2, 3])]
    assert plan.group_of_call == [0, 0, 1, 1, None, None]
    assert plan.state_calls == [4]


def test_reserve_commit_close_and_out_of_pages():
    plan = CachePlan(needs(2), 4, 4, 2)
    a = plan.open("a")
    plan.reserve(a, 9)
    assert a.tables[0] == [0, 1, 2] and a.length == 0
    plan.commit(a, 9)
    plan.reserve(a, 3)                       # 12 tokens still fit three pages
    assert a.tables[0] == [0, 1, 2]
    plan.commit(a, 3)
    b = plan.open("b")
    with pytest.raises(OutOfPages):
        plan.reserve(b, 5)                   # needs 2, one is left: nothing taken
    assert b.tables[0] == [] and plan.allocators[0].free_count == 1
    assert not plan.can_reserve(b, 5) and plan.can_reserve(b, 4)
    with pytest.raises(OutOfPages, match="request slots"):
        plan.open("c")
    plan.close(a)
    plan.reserve(b, 5)
    assert b.tables[0] == [2, 1]             # pages are used again, last freed first
    plan.check()
    plan.close(b)
    with pytest.raises(PageError, match="closed twice"):
        plan.close(b)
    assert plan.allocators[0].all_released() and plan.allocators[0].free_count == 4


def test_window_gives_pages_back_as_it_passes():
    plan = CachePlan(needs(1, 1, window=6), 16, 4, 2)
    r = plan.open("r")
    held = []
    for n in (5, 1, 1, 7, 2, 1, 1, 1, 9):
        plan.reserve(r, n)
        # every key a query of this step can see has a page
        for g, layout in enumerate(plan.groups):
            for q in range(r.length, r.length + n):
                lo = 0 if layout.window is None else max(0, q - layout.window)
                assert all(r.tables[g][k // 4] >= 0 for k in range(lo, q + 1))
        plan.commit(r, n)
        plan.check()
        held.append(len(r.pages_held(1)))
    assert len(r.pages_held(0)) == pages_for(r.length, 4)
    assert max(held) <= pages_for(6 + 9, 4) + 1 and held[-1] <= 3
    first = plan.first_needed_block(1, r.length)
    assert all(p < 0 for p in r.tables[1][:first]) and all(p >= 0 for p in r.tables[1][first:])
    plan.close(r)
    assert all(a.all_released() for a in plan.allocators)


def test_state_slots_are_unique_and_return():
    plan = CachePlan(needs(1, state=True), 4, 4, 3)
    caches = [plan.open(i) for i in range(3)]
    assert sorted(c.state_slot for c in caches) == [0, 1, 2]
    plan.close(caches[1])
    assert plan.open("again").state_slot == caches[1].state_slot
    plan.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    share = seed % 2 == 0
    window = None if share else 10
    plan = CachePlan(needs(2) if share else needs(1, 2, window=window), 24, 4, 5, share_prefixes=share)
    assert plan.share_prefixes == share
    live = {}
    base = [rng.randrange(50) for _ in range(40)]
    for step in range(400):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            name = f"q{step}"
            cache = plan.open(name)
            prompt = base[:rng.randrange(1, 30)] + [rng.randrange(50) for _ in range(rng.randrange(0, 6))]
            adopted = plan.adopt_prefix(cache, prompt[:-1])
            assert adopted % 4 == 0 and adopted <= len(prompt) - 1
            live[name] = (cache, prompt)
        elif action < 0.8 and live:
            name = rng.choice(sorted(live))
            cache, prompt = live[name]
            n = rng.randrange(1, 9)
            if cache.length < len(prompt):
                n = min(n, len(prompt) - cache.length)
            if plan.can_reserve(cache, n):
                plan.reserve(cache, n)
                plan.commit(cache, n)
                if cache.length == len(prompt):
                    plan.publish_prompt(cache, prompt)
            else:
                with pytest.raises(OutOfPages):
                    plan.reserve(cache, n)
                victim = rng.choice(sorted(live))
                if rng.random() < 0.5:
                    plan.release_pages(live[victim][0])      # preempted, recomputed later
                else:
                    plan.close(live.pop(victim)[0])
        elif live:
            plan.close(live.pop(rng.choice(sorted(live)))[0])
        plan.check()
    for cache, _ in live.values():
        plan.close(cache)
    plan.check()
    for allocator in plan.allocators:
        assert allocator.all_released() and allocator.available == allocator.capacity
        allocator.evict_kept()
        assert allocator.free_count == allocator.capacity

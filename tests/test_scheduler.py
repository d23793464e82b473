"""The scheduler's decisions, against a fake engine (no GPU): batching equals
running alone, joining, the token budget, what happens when pages run out,
failures, shared beginnings, and that every page comes back.  The cases mirror
the reference's engine tests (qwen-server/src/engine.rs:1328-1407, 1830-1963,
1965-2084, 2470-2529)."""
import pytest

from fake_engine import FakeEngine
from tokenizer_b200.engine.generate import GenerateParams, StopReason
from tokenizer_b200.engine.scheduler import Scheduler
from tiny import random_ids


def solo(prompt, params, **engine_kw):
    engine = FakeEngine(num_pages=256, **engine_kw)
    s = Scheduler(engine, max_batch_size=1, token_budget=1 << 20)
    rid = s.add_request(prompt, params)
    return s.run()[rid]


def run_checked(s):
    while s.has_work():
        s.step()
        s.cache.check()
    for a in s.cache.allocators:
        assert a.all_released() and a.available == a.capacity
    assert not s.cache.requests
    return s.finished


def test_batched_equals_solo_for_eight_requests():
    prompts = [random_ids(n, 50, 10 + n) for n in (1, 2, 3, 4, 5, 6, 9, 17)]
    params = [GenerateParams(max_tokens=3 + i, temperature=0.0) for i in range(8)]
    s = Scheduler(FakeEngine(num_pages=256), max_batch_size=8, token_budget=64)
    ids = [s.add_request(p, q) for p, q in zip(prompts, params)]
    out = run_checked(s)
    for rid, p, q in zip(ids, prompts, params):
        assert out[rid].tokens == solo(p, q).tokens
        assert out[rid].reason == StopReason.MAX_TOKENS and len(out[rid].tokens) == q.max_tokens
    assert s.stats.max_running == 8 and s.stats.preemptions == 0
    assert s.stats.requests_finished == 8


def test_sampled_requests_do_not_depend_on_the_batch():
    prompts = [random_ids(n, 50, 30 + n) for n in (5, 19, 64, 100)]
    params = [GenerateParams(max_tokens=12, temperature=0.8, top_p=0.9, seed=7 + i) for i in range(4)]
    s = Scheduler(FakeEngine(num_pages=256), max_batch_size=4, token_budget=24)
    ids = [s.add_request(p, q) for p, q in zip(prompts, params)]
    out = run_checked(s)
    for rid, p, q in zip(ids, prompts, params):
        assert out[rid].tokens == solo(p, q).tokens
    again = solo(prompts[0], params[0])
    other_seed = solo(prompts[0], GenerateParams(max_tokens=12, temperature=0.8, top_p=0.9, seed=99))
    assert again.tokens == out[ids[0]].tokens and other_seed.tokens != again.tokens


def test_token_budget_cuts_prompts_and_decodes_go_first():
    engine = FakeEngine(num_pages=256)
    s = Scheduler(engine, max_batch_size=4, token_budget=10)
    a = s.add_request(random_ids(3, 50, 1), GenerateParams(max_tokens=8))
    s.step()                                   # a's prompt runs whole
    b = s.add_request(random_ids(25, 50, 2), GenerateParams(max_tokens=2))
    run_checked(s)
    assert engine.steps[0] == [(a, 3)]
    assert engine.steps[1] == [(a, 1), (b, 9)]           # one decode, the rest of the budget
    assert engine.steps[2] == [(a, 1), (b, 9)]
    assert engine.steps[3] == [(a, 1), (b, 7)]
    assert all(sum(n for _, n in step) <= 10 for step in engine.steps)
    assert s.finished[b].tokens == solo(random_ids(25, 50, 2), GenerateParams(max_tokens=2)).tokens


def test_short_request_joins_a_running_long_one():
    engine = FakeEngine(num_pages=256)
    s = Scheduler(engine, max_batch_size=4, token_budget=64)
    long = s.add_request(random_ids(6, 50, 3), GenerateParams(max_tokens=12))
    for _ in range(4):
        s.step()
    short = s.add_request(random_ids(2, 50, 4), GenerateParams(max_tokens=3))
    finished_order = []
    while s.has_work():
        finished_order += s.step()
    assert finished_order == [short, long]
    assert s.finished[long].tokens == solo(random_ids(6, 50, 3), GenerateParams(max_tokens=12)).tokens
    assert s.stats.max_running == 2


def test_out_of_pages_preempts_the_newest_and_recomputes():
    # three pages of four tokens: two requests of prompt 3 + 6 new need 3 pages each at the end
    engine = FakeEngine(num_pages=3, page_size=4)
    s = Scheduler(engine, max_batch_size=4, token_budget=64)
    prompts = [random_ids(3, 50, 40), random_ids(3, 50, 41), random_ids(2, 50, 42)]
    ids = [s.add_request(p, GenerateParams(max_tokens=6)) for p in prompts]
    out = run_checked(s)
    for rid, p in zip(ids, prompts):
        assert out[rid].reason == StopReason.MAX_TOKENS
        assert out[rid].tokens == solo(p, GenerateParams(max_tokens=6), page_size=4).tokens
    assert s.stats.preemptions >= 1
    assert s.stats.last_preempted_id in ids[1:]          # never the oldest
    assert s.stats.peak_pages <= 3


def test_request_larger_than_the_pool_fails_and_the_next_runs():
    s = Scheduler(FakeEngine(num_pages=3, page_size=4), max_batch_size=4, token_budget=64)
    big = s.add_request(random_ids(13, 50, 5), GenerateParams(max_tokens=2))
    ok = s.add_request(random_ids(4, 50, 6), GenerateParams(max_tokens=2))
    out = run_checked(s)
    assert out[big].reason == StopReason.FAILED and "3 pages" in out[big].error
    assert out[ok].reason == StopReason.MAX_TOKENS and len(out[ok].tokens) == 2
    assert s.stats.requests_failed == 1


def test_lone_request_that_outgrows_the_pool_fails():
    s = Scheduler(FakeEngine(num_pages=2, page_size=4), max_batch_size=2, token_budget=64)
    rid = s.add_request(random_ids(6, 50, 7), GenerateParams(max_tokens=10))
    out = run_checked(s)
    assert out[rid].reason == StopReason.FAILED and len(out[rid].tokens) == 3  # 6 + 2 fill both pages


def test_shared_beginnings_use_the_same_pages_and_match_solo():
    engine = FakeEngine(num_pages=64, page_size=4, share_prefixes=True)
    s = Scheduler(engine, max_batch_size=4, token_budget=64)
    prompt = random_ids(14, 50, 8)
    first = s.add_request(prompt, GenerateParams(max_tokens=4))
    s.step()
    second = s.add_request(prompt, GenerateParams(max_tokens=4))
    third = s.add_request(prompt[:9] + [1, 2, 3], GenerateParams(max_tokens=4))
    out = run_checked(s)
    want = solo(prompt, GenerateParams(max_tokens=4), page_size=4).tokens
    assert out[first].tokens == want and out[second].tokens == want
    assert out[third].tokens == solo(prompt[:9] + [1, 2, 3], GenerateParams(max_tokens=4), page_size=4).tokens
    assert s.stats.shared_prefix_tokens == 12 + 8        # 3 full pages, then 2
    # the second copy ran only what was not shared
    assert (second, 2) in engine.steps[1]


def test_context_limit_and_empty_prompt():
    s = Scheduler(FakeEngine(num_pages=8, max_positions=16), max_batch_size=2)
    with pytest.raises(ValueError, match="max_position_embeddings"):
        s.add_request(list(range(10)), GenerateParams(max_tokens=7))
    with pytest.raises(ValueError, match="no tokens"):
        s.add_request([], GenerateParams(max_tokens=1))
    with pytest.raises(ValueError, match="temperature"):
        s.add_request([1], GenerateParams(max_tokens=1, temperature=-1.0))


def test_max_tokens_zero_runs_the_prompt_and_draws_nothing():
    engine = FakeEngine(num_pages=8)
    s = Scheduler(engine, max_batch_size=2)
    rid = s.add_request([1, 2, 3], GenerateParams(max_tokens=0))
    out = run_checked(s)
    assert out[rid].tokens == [] and out[rid].reason == StopReason.MAX_TOKENS
    assert engine.steps == [[(rid, 3)]] and s.stats.tokens_sampled == 0


def test_forward_count_is_one_prefill_plus_n_minus_one_decodes():
    engine = FakeEngine(num_pages=64)
    s = Scheduler(engine, max_batch_size=1, token_budget=1 << 20)
    s.add_request([4, 5, 6, 7, 8], GenerateParams(max_tokens=5))
    run_checked(s)
    assert len(engine.steps) == 5            # generate.rs:686-704


def test_windowed_groups_through_the_scheduler():
    from tokenizer_b200.parts.base import CacheNeed, KVNeed
    needs = [CacheNeed(kv=KVNeed(1, 8, None)), CacheNeed(kv=KVNeed(1, 8, 5))]
    engine = FakeEngine(num_pages=12, page_size=4, needs=needs)
    s = Scheduler(engine, max_batch_size=3, token_budget=16)
    prompts = [random_ids(n, 50, 60 + n) for n in (9, 14, 3)]
    ids = [s.add_request(p, GenerateParams(max_tokens=7)) for p in prompts]
    out = run_checked(s)
    for rid, p in zip(ids, prompts):
        assert out[rid].tokens == solo(p, GenerateParams(max_tokens=7), page_size=4).tokens


def test_decode_bursts_give_the_same_ids_and_fall_back_when_pages_are_short():
    """Several steps on the device between visits to the host: same ids, same reasons
    (max_tokens inside a burst, an EOS id inside a burst, a request that joins later),
    and with a pool too small for a whole burst the single steps and preemption still work."""
    prompts = [random_ids(n, 50, 70 + n) for n in (3, 8, 21, 5)]
    free = [solo(p, GenerateParams(max_tokens=14)).tokens for p in prompts]
    params = [GenerateParams(max_tokens=14), GenerateParams(max_tokens=9),
              GenerateParams(max_tokens=14, eos=[free[2][6]]), GenerateParams(max_tokens=11)]
    want = [solo(p, q) for p, q in zip(prompts, params)]
    for pages, burst in ((256, 4), (256, 5), (12, 4)):
        engine = FakeEngine(num_pages=pages)
        s = Scheduler(engine, max_batch_size=4, token_budget=16, decode_burst=burst)
        ids = [s.add_request(p, q) for p, q in zip(prompts[:3], params[:3])]
        for _ in range(3):
            s.step()
            s.cache.check()
        ids.append(s.add_request(prompts[3], params[3]))
        out = run_checked(s)
        for rid, w in zip(ids, want):
            assert out[rid].tokens == w.tokens and out[rid].reason == w.reason
            assert out[rid].completion_tokens == w.completion_tokens
        assert engine.bursts > 0
        if pages == 12:
            assert s.stats.preemptions > 0
    sampled = Scheduler(FakeEngine(num_pages=64), max_batch_size=2, token_budget=16, decode_burst=4)
    sampled.add_request(prompts[0], GenerateParams(max_tokens=6, temperature=0.7, seed=3))
    run_checked(sampled)
    assert not hasattr(sampled.engine, "bursts")          # sampled requests take single steps


def test_steps_packed_ahead_of_their_tokens_change_nothing():
    """While the ids of a step are drawn, the scheduler lets the engine pack the next
    decoding step; it is used only if exactly the same requests go on (or, where the engine
    can feed it the drawn ids on the device, launched at once and its rows for ended requests
    dropped).  Ends by EOS and
    max_tokens, a late arrival, sampled requests and a pool that forces preemption all
    give the ids of the plain path."""
    prompts = [random_ids(n, 50, 90 + n) for n in (4, 9, 17, 6)]
    free = [solo(p, GenerateParams(max_tokens=16)).tokens for p in prompts]
    params = [GenerateParams(max_tokens=16), GenerateParams(max_tokens=7),
              GenerateParams(max_tokens=16, eos=[free[2][9]]),
              GenerateParams(max_tokens=12, temperature=0.9, top_p=0.8, seed=5)]
    want = [solo(p, q) for p, q in zip(prompts, params)]
    for pages, launch in ((256, False), (11, False), (256, True), (11, True)):
        engine = FakeEngine(num_pages=pages)
        engine.enable_ahead(launch)
        s = Scheduler(engine, max_batch_size=4, token_budget=16)
        ids = [s.add_request(p, q) for p, q in zip(prompts[:3], params[:3])]
        for _ in range(4):
            s.step()
            s.cache.check()
        ids.append(s.add_request(prompts[3], params[3]))
        out = run_checked(s)
        for rid, w in zip(ids, want):
            assert out[rid].tokens == w.tokens and out[rid].reason == w.reason
        assert engine.prepared_used > 0
        # with `launch` the packed step runs on the draw's ids before the host has read them;
        # a request that ends with such an id leaves one token run for nothing
        assert (engine.launched_ahead > 0) == launch
        if pages == 11:
            assert s.stats.preemptions > 0


@pytest.mark.parametrize("seed", range(12))
def test_random_arrivals_and_ends_in_every_mode(seed):
    """Random prompts, lengths, ends (max_tokens, an end-of-sequence id from the request's own
    free run, sampled with a temperature), arrivals spread over the run and a pool that may or may
    not force preemption: single steps, steps packed ahead, steps launched on the draw's ids before
    the host has read them, and bursts all give each request the ids it gets alone, and every page
    comes back."""
    import random
    rng = random.Random(seed)
    n = rng.randint(3, 7)
    prompts = [random_ids(rng.randint(1, 30), 50, 1000 * seed + i) for i in range(n)]
    params = []
    for i, p in enumerate(prompts):
        kind = rng.choice(["max", "eos", "sampled"])
        most = rng.randint(1, 14)
        if kind == "eos":
            free = solo(p, GenerateParams(max_tokens=most)).tokens
            params.append(GenerateParams(max_tokens=most, eos=[free[rng.randrange(len(free))]]))
        elif kind == "sampled":
            params.append(GenerateParams(max_tokens=most, temperature=0.9, top_p=0.85, seed=seed * 31 + i))
        else:
            params.append(GenerateParams(max_tokens=most))
    want = [solo(p, q) for p, q in zip(prompts, params)]
    arrivals = sorted(rng.randint(0, 12) for _ in range(n))
    pages = rng.choice([256, 24, 16])          # 16 pages of 4 tokens: less than what all hold together
    for mode in ("single", "ahead", "launch", "burst"):
        engine = FakeEngine(num_pages=pages)
        if mode in ("ahead", "launch"):
            engine.enable_ahead(launch=mode == "launch")
        s = Scheduler(engine, max_batch_size=rng.choice([2, 4, 8]), token_budget=rng.choice([5, 16, 64]),
                      decode_burst=4 if mode == "burst" else 1)
        ids, at, step = [], 0, 0
        while at < n or s.has_work():
            while at < n and arrivals[at] <= step:
                ids.append(s.add_request(prompts[at], params[at]))
                at += 1
            if s.has_work():
                s.step()
                s.cache.check()
            step += 1
        for a in s.cache.allocators:
            assert a.all_released() and a.available == a.capacity
        for rid, w in zip(ids, want):
            got = s.finished[rid]
            assert got.tokens == w.tokens and got.reason == w.reason, (mode, rid)
            assert got.completion_tokens == w.completion_tokens


def test_a_batch_larger_than_the_request_slots_is_refused():
    with pytest.raises(ValueError, match="request slots"):
        Scheduler(FakeEngine(num_pages=64, max_requests=2), max_batch_size=3)


def test_the_head_waits_while_every_request_slot_is_held_elsewhere():
    """Slots held outside the scheduler (another user of the same cache): the head of the line
    waits instead of the iteration failing, and runs once a slot is free."""
    engine = FakeEngine(num_pages=64, max_requests=2)
    held = [engine.cache.open(("outside", i)) for i in range(2)]
    s = Scheduler(engine, max_batch_size=2, token_budget=64)
    prompt, params = random_ids(5, 50, 3), GenerateParams(max_tokens=4)
    rid = s.add_request(prompt, params)
    assert s.step() == [] and not s.running and len(s.waiting) == 1
    engine.cache.close(held[0])
    out = s.run()
    assert out[rid].tokens == solo(prompt, params).tokens
    engine.cache.close(held[1])
    engine.cache.check()


def test_requests_that_arrive_together_still_share_a_beginning():
    """Four requests with the same 20-token beginning arrive in one iteration, under a budget
    that lets only the first run at once.  The pages of the beginning are published as soon as
    the first request's portion has computed them, and the others, which found nothing when
    they were admitted, take them over when their own first portion comes up.  Ids equal solo."""
    engine = FakeEngine(num_pages=128, page_size=4, share_prefixes=True)
    s = Scheduler(engine, max_batch_size=4, token_budget=16)
    begin = random_ids(20, 50, 21)
    prompts = [begin + random_ids(6 + 3 * i, 50, 30 + i) for i in range(3)] + [begin + [7]]
    ids = [s.add_request(p, GenerateParams(max_tokens=5)) for p in prompts]
    out = run_checked(s)
    for rid, p in zip(ids, prompts):
        assert out[rid].tokens == solo(p, GenerateParams(max_tokens=5), page_size=4).tokens
    # the first computed the beginning itself, 16 tokens of it in its first step; the second came up
    # in the next step, when only those 16 were published; the others took over all 20
    assert s.stats.shared_prefix_tokens == 16 + 20 + 20
    assert s.stats.tokens_run == sum(len(p) + 4 for p in prompts) - 56

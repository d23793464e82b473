"""Generation through the Python entry point on the GPU: greedy ids against the
plain implementation, long decoding, the first tokens of a sequence, decoding
steps that stay on the device, and sampled requests under batching."""
import pytest
import torch

import plain_qwen2 as plain
from tiny import TINY, make_folder, random_ids

pytestmark = pytest.mark.gpu

SHARPEN = {r"\.(q|k)_proj\.weight": 8.0, r"embed_tokens|lm_head": 5.0}


@pytest.fixture(scope="module", params=["a", "b", "c"])
def folder(request, tmp_path_factory):
    return make_folder(tmp_path_factory, request.param, scale=SHARPEN)


def margins_ok(cfg, w, ids, n_prompt, least):
    """Greedy ids of two implementations can only be compared where the best
    logit leads the second by more than their rounding."""
    logits = plain.all_logits(cfg, w, ids)[n_prompt - 1:-1]
    top2 = torch.topk(logits, 2, dim=-1).values
    return bool(((top2[:, 0] - top2[:, 1]) > least).all())


def assert_near_best(cfg, w, prompt, tokens, dtype, what=""):
    """Every id is the best of the plain logits given the ids before it, up to the rounding
    of the precision (in bfloat16 two ids whose logits lie closer than that may swap)."""
    logits = plain.all_logits(cfg, w, list(prompt) + list(tokens))
    lead = logits[len(prompt) - 1:-1]
    chosen = lead.gather(1, torch.tensor(tokens)[:, None])[:, 0]
    slack = 1e-4 if dtype == "float32" else 0.04 * float(logits.abs().max())
    gap = lead.max(dim=1).values - chosen
    assert float(gap.max()) <= slack, \
        f"{what}: token {int(gap.argmax())} lies {float(gap.max())} below the best logit (slack {slack})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_equals_the_plain_implementation(folder, dtype):
    import tokenizer_b200 as tb
    path, config, page = folder
    cfg, w = plain.load_folder(path)
    model = tb.load_model(path, dtype=dtype)
    checked = 0
    for n in (1, 7, 33):
        prompt = random_ids(n, config.vocab_size, 200 + n)
        want = plain.greedy_generate(cfg, w, prompt, 16)
        out = tb.generate(model, prompt, tb.GenerateParams.greedy(16))
        assert out.reason == tb.StopReason.MAX_TOKENS and out.completion_tokens == 16
        if dtype == "float32":
            assert out.tokens == want
            checked += 1
        elif margins_ok(cfg, w, prompt + want, n, 0.05 * float(plain.all_logits(cfg, w, prompt + want).abs().max())):
            assert out.tokens == want
            checked += 1
        assert_near_best(cfg, w, prompt, out.tokens, dtype, f"prompt of {n}")
        assert tb.greedy_tokens(model, prompt, 16) == out.tokens     # the same call twice
    assert dtype == "bfloat16" or checked == 3


def test_eos_stops_generation(folder):
    import tokenizer_b200 as tb
    path, config, page = folder
    model = tb.load_model(path, dtype="float32")
    prompt = random_ids(9, config.vocab_size, 3)
    free = tb.generate(model, prompt, tb.GenerateParams.greedy(8)).tokens
    out = tb.generate(model, prompt, tb.GenerateParams(max_tokens=8, eos=[free[3]]))
    first = free.index(free[3])
    assert out.tokens == free[:first] and out.reason == tb.StopReason.EOS
    assert out.completion_tokens == first + 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_device_side_steps(folder, dtype):
    """Decode far past the prompt (many pages, the window passing pages by), one
    step at a time through the scheduler and in steps that stay on the device;
    both must give the ids of a whole-sequence recompute."""
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    path, config, page = folder
    cfg, w = plain.load_folder(path)
    n_new = min(100, config.max_position_embeddings - 12)
    prompt = random_ids(11, config.vocab_size, 77)
    model = tb.load_model(path, dtype=dtype)
    out = tb.generate(model, prompt, tb.GenerateParams.greedy(n_new)).tokens
    assert len(out) == n_new
    # every id is the argmax of the plain logits given the ids before it, up to rounding
    logits = plain.all_logits(cfg, w, prompt + out)
    lead = logits[len(prompt) - 1:-1]
    chosen = lead.gather(1, torch.tensor(out)[:, None])[:, 0]
    slack = 1e-4 if dtype == "float32" else 0.04 * float(logits.abs().max())
    worst = float((lead.max(dim=1).values - chosen).max())
    assert worst <= slack, f"token {int((lead.max(dim=1).values - chosen).argmax())} is {worst} below the best"
    # the same through decode_steps, two requests side by side
    engine = tb.engine_for(model, 2 * (len(prompt) + n_new + 64), page, max_requests=2)
    caches = [engine.cache.open(i) for i in range(2)]
    for c in caches:
        engine.cache.reserve(c, len(prompt))
    first = engine.sampler.greedy(engine.step([StepEntry(c, prompt, [len(prompt) - 1]) for c in caches])).tolist()
    assert first == [out[0], out[0]]
    ids = engine.decode_steps([StepEntry(c, [t]) for c, t in zip(caches, first)], 40)
    ids += engine.decode_steps([StepEntry(c, [t]) for c, t in zip(caches, ids[-1])], n_new - 41)
    assert [row[0] for row in ids] == [row[1] for row in ids]
    got = [out[0]] + [row[0] for row in ids]
    if dtype == "float32":
        assert got == out
    assert caches[0].length == len(prompt) + n_new - 1
    for c in caches:
        engine.cache.close(c)
    assert all(a.all_released() for a in engine.cache.allocators)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(folder, dtype):
    """Positions 0, 1, 2 alone: one key, no page filled, the rotation at angle 0."""
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    path, config, page = folder
    cfg, w = plain.load_folder(path)
    model = tb.load_model(path, dtype=dtype)
    engine = tb.engine_for(model, 64, page, max_requests=4)
    ids = random_ids(3, config.vocab_size, 9)
    want = plain.all_logits(cfg, w, ids)
    cache = engine.cache.open("x")
    rows = []
    for t in ids:
        engine.cache.reserve(cache, 1)
        rows.append(engine.step([StepEntry(cache, [t], [0])]).cpu()[0])
    bound = 1e-4 if dtype == "float32" else 2e-2 * float(want.abs().max())
    assert float((torch.stack(rows) - want).abs().max()) <= bound


def test_sampled_requests_in_a_batch_follow_their_own_draws(tmp_path_factory):
    """Config B's run: four requests of 5/19/64/100 tokens, temperature 0.8 from a
    fixed seed, portions of 24 tokens mixed with decoded tokens.  Each request's
    ids must be what its own draws select from the plain logits of its own history."""
    import tokenizer_b200 as tb
    from tokenizer_b200.sampling import uniform
    path, config, page = make_folder(tmp_path_factory, "b", scale=SHARPEN)
    cfg, w = plain.load_folder(path)
    model = tb.load_model(path, dtype="float32")
    prompts = [random_ids(n, config.vocab_size, 300 + n) for n in (5, 19, 64, 100)]
    params = [tb.GenerateParams(max_tokens=12, temperature=0.8, top_p=0.95, seed=40 + i) for i in range(4)]
    outs = tb.generate_batch(model, prompts, params, max_batch_size=4, token_budget=24, page_size=page)
    solo = [tb.generate(model, p, q) for p, q in zip(prompts, params)]
    for prompt, q, out, alone in zip(prompts, params, outs, solo):
        assert len(out.tokens) == 12 and out.tokens == alone.tokens
        logits = plain.all_logits(cfg, w, prompt + out.tokens)
        for k, token in enumerate(out.tokens):
            kept, mass = plain.sample_intervals(logits[len(prompt) - 1 + k], 0.8, 0.95)
            assert token in kept
            at, total = kept.index(token), sum(mass)
            u = uniform(q.seed, k)
            assert sum(mass[:at]) - 1e-4 * total <= u * total < sum(mass[:at + 1]) + 1e-4 * total


def test_the_engine_refuses_what_it_cannot_run(folder):
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    path, config, page = folder
    model = tb.load_model(path, dtype="float32")
    engine = tb.engine_for(model, 64, page, max_requests=2)
    cache = engine.cache.open("x")
    with pytest.raises(ValueError, match="no pages reserved"):
        engine.step([StepEntry(cache, [1, 2], [0])])
    engine.cache.reserve(cache, 2)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        engine.step([StepEntry(cache, [1, config.vocab_size], [0])])
    with pytest.raises(ValueError, match="wanted place"):
        engine.step([StepEntry(cache, [1, 2], [2])])
    with pytest.raises(ValueError, match="twice"):
        engine.step([StepEntry(cache, [1], [0]), StepEntry(cache, [2], [0])])
    with pytest.raises(Exception, match="GPU"):
        tb.load_model(path, dtype="float32", device="cpu")
    assert engine.step([StepEntry(cache, [1, 2], [1])]).shape == (1, config.vocab_size)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scheduler_on_the_engine_with_too_few_pages(folder, dtype):
    """Continuous batching on the real engine with a pool so small that requests are
    preempted and recomputed: every request still gets the ids it gets alone, and
    every page comes back."""
    import tokenizer_b200 as tb
    from tokenizer_b200.engine.scheduler import Scheduler
    path, config, page = folder
    cfg, w = plain.load_folder(path)
    model = tb.load_model(path, dtype=dtype)
    lengths = [9, 30, 17, 44, 5]
    new = 20
    prompts = [random_ids(n, config.vocab_size, 500 + n) for n in lengths]
    solo = [tb.generate(model, p, tb.GenerateParams.greedy(new)).tokens for p in prompts]
    # room for about two and a half of the five requests at their final length
    total = sum(-(-(n + new) // page) for n in lengths)
    engine = tb.Engine(model, num_pages=max(total // 2, -(-(max(lengths) + new) // page) + 1),
                       page_size=page, max_requests=4, share_prefixes=False)
    scheduler = Scheduler(engine, max_batch_size=4, token_budget=24)
    ids = [scheduler.add_request(p, tb.GenerateParams.greedy(new)) for p in prompts]
    results = scheduler.run()
    assert scheduler.stats.preemptions > 0
    for rid, want, prompt in zip(ids, solo, prompts):
        assert results[rid].reason == tb.StopReason.MAX_TOKENS
        assert len(results[rid].tokens) == new
        if dtype == "float32":
            assert results[rid].tokens == want
        # a context recomputed after a preemption must still lead to ids the plain logits back
        assert_near_best(cfg, w, prompt, results[rid].tokens, dtype, f"request {rid}")
    engine.cache.check()
    assert all(a.all_released() and a.available == a.capacity for a in engine.cache.allocators)


def test_shared_beginnings_on_the_engine(folder):
    """Two requests with the same long beginning: the second adopts the first's
    full pages, runs only its own tail, and gets the ids it gets alone."""
    import tokenizer_b200 as tb
    from tokenizer_b200.engine.scheduler import Scheduler
    path, config, page = folder
    if any(l.mixer.params["window"] is not None for l in config.model_spec().layers):
        pytest.skip("pages are shared only when every layer keeps all keys")
    model = tb.load_model(path, dtype="float32")
    base = random_ids(3 * page + 5, config.vocab_size, 901)
    a, b = base + [1, 2, 3], base + [4, 5]
    alone = [tb.generate(model, p, tb.GenerateParams.greedy(6)).tokens for p in (a, b)]
    engine = tb.Engine(model, num_pages=64, page_size=page, max_requests=4, share_prefixes=True)
    scheduler = Scheduler(engine, max_batch_size=4, token_budget=512)
    first = scheduler.add_request(a, tb.GenerateParams.greedy(6))
    scheduler.step()
    second = scheduler.add_request(b, tb.GenerateParams.greedy(6))
    results = scheduler.run()
    assert scheduler.stats.shared_prefix_tokens == 3 * page
    assert results[first].tokens == alone[0] and results[second].tokens == alone[1]
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_shared_pages_are_read_and_never_rewritten(folder, dtype):
    """A second and a third request take over the published pages of a first: their logits
    behind the shared beginning are the plain ones, and what the shared pages hold, in every
    layer, is bit for bit what the first request wrote (the reference snapshots a shared
    block around the second sharer's run in the same way: qwen-server/src/engine.rs:2208-2320)."""
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    path, config, page = folder
    if any(l.mixer.params["window"] is not None for l in config.model_spec().layers):
        pytest.skip("pages are shared only when every layer keeps all keys")
    cfg, w = plain.load_folder(path)
    model = tb.load_model(path, dtype=dtype)
    engine = tb.Engine(model, num_pages=40, page_size=page, max_requests=4, share_prefixes=True)
    base = random_ids(3 * page + 5, config.vocab_size, 911)
    first = engine.cache.open("first")
    engine.cache.reserve(first, len(base))
    engine.step([StepEntry(first, base, [])])
    engine.cache.publish_prompt(first, base)
    shared_pages = list(first.tables[0][:3])

    def snapshot():
        pool = engine.cache.pools[0]            # [calls, 2, pages * page, kv heads, head size]
        return torch.stack([pool[:, :, p * page:(p + 1) * page].clone() for p in shared_pages])

    before = snapshot()
    bound_of = lambda want: 1e-4 if dtype == "float32" else 2e-2 * float(want.abs().max())
    for name, tail in (("second", [1, 2, 3, 4, 5, 6, 7]), ("third", random_ids(2 * page + 3, config.vocab_size, 5))):
        ids = base + tail
        want = plain.all_logits(cfg, w, ids)
        cache = engine.cache.open(name)
        adopted = engine.cache.adopt_prefix(cache, ids[:-1])
        assert adopted == 3 * page and cache.tables[0][:3] == shared_pages
        cut = adopted + 4                        # a portion that starts right behind the shared pages
        engine.cache.reserve(cache, cut - adopted)
        got = [engine.step([StepEntry(cache, ids[adopted:cut], list(range(cut - adopted)))]).float().cpu()]
        for t in ids[cut:]:                      # then token by token, beside the first request's decoding
            engine.cache.reserve(cache, 1)
            engine.cache.reserve(first, 1)
            got.append(engine.step([StepEntry(cache, [t], [0]), StepEntry(first, [t], [])]).float().cpu())
        err = float((torch.cat(got) - want[adopted:]).abs().max())
        assert err <= bound_of(want), f"{name}: {err}"
        assert torch.equal(snapshot(), before), f"{name} changed a shared page"
    engine.cache.check()
    for name in ("second", "third", "first"):
        engine.cache.close(engine.cache.requests[name])
    assert all(a.live == 0 for a in engine.cache.allocators)


@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
def test_long_portions_on_either_prompt_kernel(tmp_path_factory, monkeypatch, kernel):
    """Heads of 64 and portions of more than a hundred tokens reach the tensor-core
    kernels for prompts; either of the two (mma.sync tiles of 64 rows, tcgen05 tiles of
    128 rows) must give the plain logits, cut in portions that end inside a tile."""
    import tokenizer_b200 as tb
    from tokenizer_b200 import Qwen2Config, write_random_model
    from tokenizer_b200.engine import StepEntry
    from tokenizer_b200.parts import attention
    monkeypatch.setattr(attention, "_PROMPT_KERNEL", kernel)
    config = Qwen2Config.from_dict(dict(
        architectures=["Qwen2ForCausalLM"], hidden_act="silu", num_hidden_layers=2, hidden_size=128,
        num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=256, vocab_size=333,
        rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=1024,
        use_sliding_window=False, sliding_window=None, max_window_layers=2))
    path = str(tmp_path_factory.mktemp("tiny_long"))
    write_random_model(path, config, 5, scale=SHARPEN)
    cfg, w = plain.load_folder(path)
    ids = random_ids(421, config.vocab_size, 17)
    want = plain.all_logits(cfg, w, ids)
    model = tb.load_model(path, dtype="bfloat16")
    engine = tb.engine_for(model, 512, 16, max_requests=2)
    cache = engine.cache.open("x")
    got, at = [], 0
    for n in (150, 131, 140):
        engine.cache.reserve(cache, n)
        got.append(engine.step([StepEntry(cache, ids[at:at + n], list(range(n)))]).float().cpu())
        at += n
    bound = 2e-2 * float(want.abs().max())
    assert float((torch.cat(got) - want).abs().max()) <= bound


def test_decode_bursts_on_the_engine(folder):
    """Greedy requests run several steps on the device between visits to the host;
    ids, reasons and counts equal those of single steps (one request ends by
    max_tokens inside a burst, one by an EOS id)."""
    import tokenizer_b200 as tb
    path, config, page = folder
    model = tb.load_model(path, dtype="float32")
    prompts = [random_ids(n, config.vocab_size, 700 + n) for n in (6, 23, 40)]
    free = tb.generate(model, prompts[2], tb.GenerateParams.greedy(20)).tokens
    params = [tb.GenerateParams.greedy(21), tb.GenerateParams.greedy(10),
              tb.GenerateParams(max_tokens=20, eos=[free[9]])]
    single = tb.generate_batch(model, prompts, params, max_batch_size=3, page_size=page)
    burst = tb.generate_batch(model, prompts, params, max_batch_size=3, page_size=page, decode_burst=8)
    for a, b in zip(single, burst):
        assert a.tokens == b.tokens and a.reason == b.reason
        assert a.completion_tokens == b.completion_tokens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_fed_with_the_draw_on_the_device(folder, dtype):
    """Once a decoding shape is captured, the scheduler launches the next step with the ids the
    sampler has just drawn, before the host has read them.  Ids, reasons and counts equal those
    of the same batch stepped only after the host has read each draw: one request ends by an
    end-of-sequence id (its extra token is dropped and the batch shrinks), one by max_tokens;
    in 32-bit a third is sampled with a temperature, and every request equals itself alone."""
    import tokenizer_b200 as tb
    path, config, page = folder
    model = tb.load_model(path, dtype=dtype)
    prompts = [random_ids(n, config.vocab_size, 900 + n) for n in (5, 19, 33)]
    free = tb.generate(model, prompts[1], tb.GenerateParams.greedy(30)).tokens
    last = tb.GenerateParams(max_tokens=25, temperature=0.8, top_p=0.9, seed=11) if dtype == "float32" \
        else tb.GenerateParams.greedy(25)
    params = [tb.GenerateParams.greedy(40), tb.GenerateParams(max_tokens=30, eos=[free[17]]), last]
    fed = tb.engine_for(model, 64 * 3 + 64, page, max_requests=3)
    together = tb.generate_batch(fed, prompts, params, max_batch_size=3, page_size=page)
    waiting = tb.engine_for(model, 64 * 3 + 64, page, max_requests=3)
    waiting.step_prepared_device = lambda prepared, pending: None
    stepwise = tb.generate_batch(waiting, prompts, params, max_batch_size=3, page_size=page)
    for a, b in zip(stepwise, together):
        assert a.tokens == b.tokens and a.reason == b.reason
        assert a.completion_tokens == b.completion_tokens
    if dtype == "float32":
        for p, q, b in zip(prompts, params, together):
            assert tb.generate(model, p, q).tokens == b.tokens
    assert together[1].reason == tb.StopReason.EOS and len(together[1].tokens) == free.index(free[17])
    assert fed.steps_fed_on_device > 20 and waiting.steps_fed_on_device == 0
    assert all(a.live == 0 for a in fed.cache.allocators)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_of_a_captured_shape_are_replayed_with_other_contents(tmp_path_factory, dtype):
    """Steps that bring a whole number of 128-token tiles, or a few rows less (the rest are
    idle rows), are captured once per shape and replayed: the first use runs plainly, the
    second captures, later ones replay.  Each use here cuts its 249 to 256 tokens
    differently (two portions; a long portion beside a decoding token of an older request)
    and must give the plain logits."""
    import tokenizer_b200 as tb
    from tokenizer_b200 import Qwen2Config, write_random_model
    from tokenizer_b200.engine import StepEntry
    config = Qwen2Config.from_dict(dict(
        architectures=["Qwen2ForCausalLM"], hidden_act="silu", num_hidden_layers=2, hidden_size=128,
        num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=256, vocab_size=333,
        rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=1024,
        use_sliding_window=False, sliding_window=None, max_window_layers=2))
    path = str(tmp_path_factory.mktemp("tiny_shapes"))
    write_random_model(path, config, 6, scale=SHARPEN)
    cfg, w = plain.load_folder(path)
    model = tb.load_model(path, dtype=dtype)
    engine = tb.engine_for(model, 2048, 16, max_requests=4)
    old = engine.cache.open("old")
    old_ids = random_ids(42, config.vocab_size, 1)
    old_want = plain.all_logits(cfg, w, old_ids)
    engine.cache.reserve(old, 39)
    engine.step([StepEntry(old, old_ids[:39], [])])
    old_at = 39
    for use, (n_a, n_b) in enumerate(((150, 106), (100, 156), (255, 0), (131, 125), (140, 109), (251, 0))):
        a_ids = random_ids(n_a, config.vocab_size, 10 + use)
        a = engine.cache.open(("a", use))
        engine.cache.reserve(a, n_a)
        entries = [StepEntry(a, a_ids, [n_a - 1, 0])]
        wants = [plain.all_logits(cfg, w, a_ids)[[n_a - 1, 0]]]
        if n_b:
            b_ids = random_ids(n_b, config.vocab_size, 20 + use)
            b = engine.cache.open(("b", use))
            engine.cache.reserve(b, n_b)
            entries.append(StepEntry(b, b_ids, []))
        else:
            engine.cache.reserve(old, 1)                      # one decoded token beside the portion
            entries.append(StepEntry(old, old_ids[old_at:old_at + 1], [0]))
            wants.append(old_want[[old_at]])
            old_at += 1
        got = engine.step(entries).float().cpu()
        want = torch.cat(wants)
        bound = 1e-4 if dtype == "float32" else 2e-2 * float(want.abs().max())
        assert float((got - want).abs().max()) <= bound, f"use {use}"
        for e in entries:
            if e.cache is not old:
                engine.cache.close(e.cache)
    assert any(k[0] == "portions" and "graph" in v for k, v in engine._graphs.items())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_steps_are_captured_and_replayed(tmp_path_factory, dtype):
    """Steps of a few tokens to a few dozen (a short prompt, a long one's last portion, alone or
    beside a decoding token) are captured per padded shape (whole 16 rows under 64, whole 64 under
    256) and replayed: three uses of each shape with other contents and other cuts, each against
    the plain logits."""
    import tokenizer_b200 as tb
    from tokenizer_b200 import Qwen2Config, write_random_model
    from tokenizer_b200.engine import StepEntry
    config = Qwen2Config.from_dict(dict(
        architectures=["Qwen2ForCausalLM"], hidden_act="silu", num_hidden_layers=2, hidden_size=128,
        num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=256, vocab_size=333,
        rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=1024,
        use_sliding_window=False, sliding_window=None, max_window_layers=2))
    path = str(tmp_path_factory.mktemp("tiny_short_steps"))
    write_random_model(path, config, 8, scale=SHARPEN)
    cfg, w = plain.load_folder(path)
    model = tb.load_model(path, dtype=dtype)
    engine = tb.engine_for(model, 4096, 16, max_requests=4)
    old = engine.cache.open("old")
    old_ids = random_ids(80, config.vocab_size, 1)
    old_want = plain.all_logits(cfg, w, old_ids)
    engine.cache.reserve(old, 30)
    engine.step([StepEntry(old, old_ids[:30], [])])
    old_at = 30
    use = 0
    for total, with_decode in ((37, False), (90, False), (7, False), (150, True), (21, True), (200, False)):
        for rep in range(3):
            use += 1
            n_a = total - (3 + rep if total > 40 else 0)            # another cut every time, the same padded shape
            a_ids = random_ids(n_a, config.vocab_size, 100 + use)
            a = engine.cache.open(("a", use))
            engine.cache.reserve(a, n_a)
            entries = [StepEntry(a, a_ids, [n_a - 1])]
            wants = [plain.all_logits(cfg, w, a_ids)[[n_a - 1]]]
            if with_decode:
                engine.cache.reserve(old, 1)
                entries.append(StepEntry(old, old_ids[old_at:old_at + 1], [0]))
                wants.append(old_want[[old_at]])
                old_at += 1
            got = engine.step(entries).float().cpu()
            want = torch.cat(wants)
            bound = 1e-4 if dtype == "float32" else 2e-2 * float(want.abs().max())
            assert float((got - want).abs().max()) <= bound, f"{total} tokens, use {rep}"
            engine.cache.close(a)
    engine.check()
    padded = sorted({k[1] for k, v in engine._graphs.items() if k[0] == "portions" and "graph" in v})
    assert padded == [16, 32, 48, 128, 192, 256], padded


def test_logits_of_a_replayed_step_live_until_the_next_step(tmp_path_factory):
    """`Engine.step` says that its logits are valid until the engine's next step: a step replayed
    from a captured graph returns a view of the graph's output buffer.  Held across the next replay
    of the same shape they show that step's values; a clone keeps its own."""
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    path, config, page = make_folder(tmp_path_factory, "a", scale=SHARPEN)
    engine = tb.engine_for(tb.load_model(path, dtype="bfloat16"), 128, page, max_requests=1)
    cache = engine.cache.open("x")
    ids = random_ids(8, config.vocab_size, 4)
    kept = []
    for t in ids:                                 # the shape's first step runs plainly, the second is captured
        engine.cache.reserve(cache, 1)
        logits = engine.step([StepEntry(cache, [t], [0])])
        kept.append((logits, logits.clone()))
    views = [view for view, _ in kept[3:]]        # replays: the same buffer every time
    assert all(v.data_ptr() == views[0].data_ptr() for v in views)
    assert torch.equal(views[0], kept[-1][1])     # an old view shows the last step's logits ...
    assert not torch.equal(kept[3][1], kept[-1][1])            # ... which its clone does not

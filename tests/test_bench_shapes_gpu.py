"""The shapes that the benchmark times, through `Engine`, against the plain logits: decoding
with 16, 32 and 64 live requests of unequal lengths; one step of 2,048 prompt tokens (one
request, and three requests side by side) run plainly, captured and replayed; block tables
wider than 64 pages beside short ones; a burst of device-side steps that ends exactly on a
table's last slot.  Real widths with few layers keep the plain forward cheap; every request's
prompt is a beginning of one id sequence, so one plain forward serves them all."""
import pytest
import torch

import plain_qwen2 as plain
from tiny import random_ids

pytestmark = pytest.mark.gpu

WIDTHS = {
    # Qwen2.5-0.5B layer sizes (head size 64), a vocabulary that is no power of two
    "0.5B": dict(num_hidden_layers=2, hidden_size=896, num_attention_heads=14, num_key_value_heads=2,
                 intermediate_size=4864, vocab_size=32003, tie_word_embeddings=True),
    # Qwen2.5-1.5B layer sizes (head size 128)
    "1.5B": dict(num_hidden_layers=1, hidden_size=1536, num_attention_heads=12, num_key_value_heads=2,
                 intermediate_size=8960, vocab_size=20011, tie_word_embeddings=False),
    # narrow layers for long contexts (the plain attention is quadratic in memory)
    "narrow": dict(num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                   intermediate_size=512, vocab_size=1000, tie_word_embeddings=False),
}


def make_model(tmp_path_factory, widths, max_positions, seed=11):
    import tokenizer_b200 as tb
    sizes = WIDTHS[widths]
    config = tb.Qwen2Config.from_dict(dict(
        sizes, architectures=["Qwen2ForCausalLM"], hidden_act="silu", rope_theta=1000000.0,
        rms_norm_eps=1e-6, max_position_embeddings=max_positions, use_sliding_window=False,
        sliding_window=max_positions, max_window_layers=sizes["num_hidden_layers"]))
    path = str(tmp_path_factory.mktemp(f"shapes_{widths}"))
    tb.write_random_model(path, config, seed)
    cfg, w = plain.load_folder(path)
    return path, config, cfg, w


def bound_for(dtype, want):
    return 1e-4 if dtype == "float32" else 2e-2 * float(want.abs().max())


def check_rows(got, want_rows, dtype, what, scale_of):
    err = (got.float().cpu() - want_rows).abs().max(dim=1).values
    bound = bound_for(dtype, scale_of)
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    assert float(err.max()) <= bound, f"{what}: wanted row {int(err.argmax())} is off by {float(err.max()):.4g} (allowed {bound:.4g})"


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("widths", ["0.5B", "1.5B"])
def test_decoding_with_many_live_requests(tmp_path_factory, widths, dtype):
    """16, 32 and 64 requests of unequal lengths decoded together: three steps through
    `Engine.step` (the shape's first step runs plainly, the second is captured, the third
    replayed) against the plain logits, then steps that stay on the device against the same
    steps taken one by one."""
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    path, config, cfg, w = make_model(tmp_path_factory, widths, 1024)
    ids = random_ids(340, config.vocab_size, 5)
    want = plain.all_logits(cfg, w, ids)
    model = tb.load_model(path, dtype=dtype)
    for batch in (16, 32, 64) if widths == "0.5B" else (32,):
        lengths = [17 + (37 * i) % 290 for i in range(batch)]
        assert len(set(lengths)) > batch // 2

        def prefilled():
            engine = tb.engine_for(model, batch * 352, 16, max_requests=batch, share_prefixes=False)
            caches = [engine.cache.open(i) for i in range(batch)]
            for lo in range(0, batch, 8):
                for c, n in zip(caches[lo:lo + 8], lengths[lo:lo + 8]):
                    engine.cache.reserve(c, n)
                got = engine.step([StepEntry(c, ids[:n], [n - 1])
                                   for c, n in zip(caches[lo:lo + 8], lengths[lo:lo + 8])])
                check_rows(got, want[[n - 1 for n in lengths[lo:lo + 8]]], dtype,
                           f"batch {batch}: prompts {lo}..", want)
            return engine, caches

        engine, caches = prefilled()
        for step in range(3):
            for c in caches:
                engine.cache.reserve(c, 1)
            got = engine.step([StepEntry(c, [ids[n + step]], [0]) for c, n in zip(caches, lengths)])
            check_rows(got, want[[n + step for n in lengths]], dtype, f"batch {batch}: decoding step {step}", want)
        assert any(len(k) == 2 and "graph" in v for k, v in engine._graphs.items()), "the step was not captured"
        # four steps on the device: the first draw is backed by the plain logits, and all of
        # them equal the same steps taken one at a time on a second engine
        start = [n + 3 for n in lengths]
        drawn = engine.decode_steps([StepEntry(c, [ids[n]]) for c, n in zip(caches, start)], 4)
        top2 = torch.topk(want[start], 2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > 2 * bound_for(dtype, want)
        assert int(clear.sum()) >= 3
        for i in range(batch):
            if clear[i]:
                assert drawn[0][i] == int(want[start[i]].argmax()), f"batch {batch}: row {i} of the first device-side step"
        other, others = prefilled()
        tokens = None
        for step in range(3 + 4):
            for c in others:
                other.cache.reserve(c, 1)
            feed = [ids[n + step] for n in lengths] if step <= 3 else tokens
            logits = other.step([StepEntry(c, [t], [0]) for c, t in zip(others, feed)])
            tokens = other.sampler.greedy(logits).tolist()
            if step >= 3:
                assert tokens == drawn[step - 3], f"batch {batch}: device-side step {step - 3} differs from the single step"
        engine.check()
        del engine, other
        torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype,products", [("bfloat16", ""), ("bfloat16", "own"), ("float32", "")])
def test_a_step_of_2048_prompt_tokens(tmp_path_factory, monkeypatch, dtype, products):
    """The benchmark's prompt step: 2,048 tokens of one request, and of three requests
    (700 + 700 + 648), each shape three times over with other contents (run plainly, captured,
    replayed), against the plain logits at rows around every tile edge.  In bfloat16 once as
    served (plain products of many rows from the vendor library) and once with every product on
    the framework's own tensor-core kernels (tiles on pairs of CTAs, products cut along k)."""
    if products:
        monkeypatch.setenv("TOKB200_GEMM", products)
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    path, config, cfg, w = make_model(tmp_path_factory, "0.5B", 4096)
    sequences = [random_ids(2048, config.vocab_size, 21 + k) for k in range(2)]
    rows = [0, 1, 63, 64, 127, 128, 129, 255, 256, 647, 648, 699, 700, 1023, 1024, 1500, 2046, 2047]
    wants = [plain.all_logits(cfg, w, s, rows=rows) for s in sequences]
    at = {r: i for i, r in enumerate(rows)}
    model = tb.load_model(path, dtype=dtype)
    engine = tb.engine_for(model, 2048 + 64, 16, max_requests=4, share_prefixes=False)
    # a step is replayed from a captured graph only when it wants no more rows than it has
    # requests (rounded up to a power of two), as a scheduler's steps do: the first use of each
    # cut wants many rows and runs plainly, the next three want one row a request
    for use in range(4):
        which = use % 2
        mine = rows if use == 0 else [[2047], [128], [1023]][use - 1]
        cache = engine.cache.open(("one", use))
        engine.cache.reserve(cache, 2048)
        got = engine.step([StepEntry(cache, sequences[which], mine)])
        check_rows(got, wants[which][[at[r] for r in mine]], dtype, f"one request, use {use}", wants[which])
        engine.cache.close(cache)
    cuts = [(0, 700), (1, 700), (0, 648)]
    for use in range(4):
        order = cuts[use % 3:] + cuts[:use % 3]
        entries, want_rows = [], []
        for k, (which, n) in enumerate(order):
            cache = engine.cache.open(("three", use, k))
            engine.cache.reserve(cache, n)
            mine = ([r for r in rows if r < n][-4:] + [0]) if use == 0 else [[647, 128, 0][(use + k) % 3]]
            entries.append(StepEntry(cache, sequences[which][:n], mine))
            want_rows.append(wants[which][[at[r] for r in mine]])
        got = engine.step(entries)
        check_rows(got, torch.cat(want_rows), dtype, f"three requests, use {use}", wants[0])
        for e in entries:
            engine.cache.close(e.cache)
    if engine.use_graphs:
        assert sum(1 for k, v in engine._graphs.items() if k[0] == "portions" and "graph" in v) == 2
    engine.check()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_block_tables_wider_than_64_pages(tmp_path_factory, dtype):
    """Requests of 1,500 and 4,200 tokens (94 and 263 pages of 16: captured table widths of 128
    and 320) decoded beside requests of 30 and 200 tokens, alone and together, through single
    steps and device-side steps."""
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    path, config, cfg, w = make_model(tmp_path_factory, "narrow", 8192)
    ids = random_ids(4210, config.vocab_size, 31)
    lengths = [4200, 30, 1500, 200]
    rows = sorted({n - 1 + k for n in lengths for k in range(0, 8)})
    want = plain.all_logits(cfg, w, ids, rows=rows)
    at = {r: i for i, r in enumerate(rows)}
    model = tb.load_model(path, dtype=dtype)
    engine = tb.engine_for(model, sum(-(-(n + 16) // 16) * 16 for n in lengths), 16, max_requests=4,
                           share_prefixes=False)
    caches = [engine.cache.open(i) for i in range(4)]
    for c, n in zip(caches, lengths):
        done = 0
        while done < n:                       # prompts in portions of up to 2,048 tokens
            take = min(2048, n - done)
            engine.cache.reserve(c, take)
            got = engine.step([StepEntry(c, ids[done:done + take], [take - 1] if done + take == n else [])])
            done += take
        check_rows(got, want[[at[n - 1]]], dtype, f"prompt of {n}", want)
    # the long ones alone (width 320), then with the others (same width, more rows)
    for step in range(2):
        engine.cache.reserve(caches[0], 1)
        got = engine.step([StepEntry(caches[0], [ids[4200 + step]], [0])])
        check_rows(got, want[[at[4200 + step]]], dtype, f"4,200 alone, step {step}", want)
    lengths[0] += 2
    for step in range(3):
        for c in caches:
            engine.cache.reserve(c, 1)
        where = [n + step for n in lengths]
        got = engine.step([StepEntry(c, [ids[p]], [0]) for c, p in zip(caches, where)])
        check_rows(got, want[[at[p] for p in where]], dtype, f"four together, step {step}", want)
    assert any(len(k) == 2 and k[1][0] == 320 for k in engine._graphs)
    # device-side steps at these widths: the first draw against the plain logits
    where = [n + 3 for n in lengths]
    drawn = engine.decode_steps([StepEntry(c, [ids[p]]) for c, p in zip(caches, where)], 2)
    for i, p in enumerate(where):
        top2 = torch.topk(want[at[p]], 2).values
        if float(top2[0] - top2[1]) > 2 * bound_for(dtype, want):
            assert drawn[0][i] == int(want[at[p]].argmax()), f"request {i}"
    engine.check()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_device_side_steps_that_end_on_a_table_s_last_slot(tmp_path_factory, dtype):
    """A burst whose last token fills the last slot of the captured table width (8 pages of 16:
    a final length of 128): after it the next position lies outside the table, which the
    device-side advance must not read.  Ids equal those of single steps."""
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    path, config, cfg, w = make_model(tmp_path_factory, "narrow", 8192)
    model = tb.load_model(path, dtype=dtype)
    prompts = [random_ids(n, config.vocab_size, 40 + n) for n in (119, 60)]
    alone = [tb.generate(model, p, tb.GenerateParams.greedy(10)).tokens for p in prompts]
    engine = tb.engine_for(model, 2 * 128, 16, max_requests=2, share_prefixes=False)
    caches = [engine.cache.open(i) for i in range(2)]
    for c, p in zip(caches, prompts):
        engine.cache.reserve(c, len(p))
    first = engine.sampler.greedy(engine.step([StepEntry(c, p, [len(p) - 1]) for c, p in zip(caches, prompts)])).tolist()
    drawn = engine.decode_steps([StepEntry(c, [t]) for c, t in zip(caches, first)], 4)
    drawn += engine.decode_steps([StepEntry(c, [t]) for c, t in zip(caches, drawn[-1])], 5)
    assert caches[0].length == 128 and len(caches[0].tables[0]) == 8
    got = [[first[i]] + [row[i] for row in drawn] for i in range(2)]
    if dtype == "float32":
        assert got == alone
    else:
        assert [g[0] for g in got] == [a[0] for a in alone]
    engine.check()

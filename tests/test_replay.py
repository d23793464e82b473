"""Replay through bin/trace_run against the plain implementation: the same
requests whole, with the last 32 tokens decoded one by one, in portions of
changing size, and mixed with other requests on so few pages that they are
used again, in float32 and in bfloat16."""
import pytest

import replay_util as ru
from tiny import TINY, make_folder, random_ids

pytestmark = pytest.mark.gpu

SHARPEN = {r"\.(q|k)_proj\.weight": 8.0, r"embed_tokens|lm_head": 5.0}
LENGTHS = {"a": [1, 7, 33, 100, 128, 65], "b": [5, 19, 64, 100, 200, 131], "c": [3, 40, 97, 150, 260, 64]}


@pytest.fixture(scope="module", params=sorted(TINY))
def model(request, tmp_path_factory):
    folder, config, page = make_folder(tmp_path_factory, request.param, scale=SHARPEN)
    requests = {f"r{i}": random_ids(n, config.vocab_size, 100 + i)
                for i, n in enumerate(LENGTHS[request.param])}
    return folder, config, page, requests, ru.reference_logits(folder, requests)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole(model, dtype, tmp_path):
    folder, config, page, requests, want = model
    steps = ru.steps_whole(requests)
    budget = max(ru.rounded64(len(v)) for v in requests.values())
    got = ru.collect(steps, ru.run_trace(folder, dtype, steps, str(tmp_path), budget, page))
    assert {k: len(v) for k, v in got.items()} == {k: len(v) for k, v in requests.items()}
    ru.compare(got, want, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_tokens_one_by_one(model, dtype, tmp_path):
    folder, config, page, requests, want = model
    steps = ru.steps_decode_tail(requests, 32)
    budget = max(ru.rounded64(len(v)) for v in requests.values())
    got = ru.collect(steps, ru.run_trace(folder, dtype, steps, str(tmp_path), budget, page))
    ru.compare(got, want, dtype, "decode tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_changing_size(model, dtype, tmp_path):
    folder, config, page, requests, want = model
    steps = ru.steps_portions(requests)
    budget = max(ru.rounded64(len(v)) for v in requests.values())
    got = ru.collect(steps, ru.run_trace(folder, dtype, steps, str(tmp_path), budget, page))
    assert {k: len(v) for k, v in got.items()} == {k: len(v) for k, v in requests.items()}
    ru.compare(got, want, dtype, "portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_with_page_reuse(model, dtype, tmp_path):
    folder, config, page, requests, want = model
    steps, peak = ru.steps_mixed(requests, max_live=4)
    total = sum(ru.rounded64(len(v)) for v in requests.values())
    assert peak < total, "the trace must force pages to be used again"
    got = ru.collect(steps, ru.run_trace(folder, dtype, steps, str(tmp_path), peak, page))
    assert {k: len(v) for k, v in got.items()} == {k: len(v) for k, v in requests.items()}
    ru.compare(got, want, dtype, "mixed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_with_shared_pages(model, dtype, tmp_path):
    """As above, and two of the requests begin with the first tokens of another that is still
    running: they take its published pages over instead of computing them, while pages of
    ended requests are used again around them.  The logits behind the shared pages must be
    what the plain implementation gives for the whole sequence."""
    folder, config, page, requests, want = model
    if config.use_sliding_window:
        pytest.skip("a cache with a windowed group shares no pages")
    names = sorted(requests)
    donor = max(names, key=lambda n: len(requests[n]))
    shared = (len(requests[donor]) * 2 // 3) // page * page
    assert shared >= 2 * page
    requests = dict(requests)
    extra = {}
    for k, n_shared in enumerate((shared, shared - page)):
        tail = random_ids(23 + 9 * k, config.vocab_size, 900 + k)
        extra[f"s{k}"] = requests[donor][:n_shared] + tail
    # the donor first, then one other, then the two sharers, then the rest
    others = [n for n in names if n != donor]
    ordered = {donor: requests[donor], others[0]: requests[others[0]]}
    ordered.update(extra)
    ordered.update({n: requests[n] for n in others[1:]})
    share = {"s0": (donor, shared), "s1": (donor, shared - page)}
    want = dict(want)
    want.update(ru.reference_logits(folder, extra))
    steps, peak, expect = ru.steps_mixed(ordered, max_live=4, share=share, page=page)
    assert all(n >= 2 * page or n == shared - page for n in expect.values()) and min(expect.values()) >= page
    adopted = {}
    got = ru.collect(steps, ru.run_trace(folder, dtype, steps, str(tmp_path), peak, page,
                                         share=True, adopted=adopted))
    assert adopted == expect, f"pages were not shared as planned: {adopted} vs {expect}"
    for name, ids in ordered.items():
        assert len(got[name]) == len(ids) - expect.get(name, 0)
    ru.compare(got, want, dtype, "mixed with shared pages")

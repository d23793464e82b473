"""What the host packs for a step (no GPU): a step of single tokens is written column by column,
any other step entry by entry; for single tokens both ways must fill the buffer alike.  Also what
`validate` refuses."""
import random

import numpy as np
import pytest
import torch

from tokenizer_b200.cache import CachePlan
from tokenizer_b200.engine import batch as batch_module
from tokenizer_b200.engine.batch import BatchBuilder, StepEntry
from tokenizer_b200.parts.attention import RowTiles
from tokenizer_b200.parts.base import BatchAnnotation, CacheNeed, KVNeed


class LongestFirst(BatchAnnotation):
    """An annotation defined here: the requests in the order of their stored lengths."""
    key = "longest_first"

    def capacity(self, n_tokens, n_requests):
        return n_requests

    def fill(self, out, first_rows, counts, starts, padded):
        order = np.argsort(-(starts + counts), kind="stable")
        out[:len(order)] = order
        return len(order)


NOTES = [RowTiles(64), RowTiles(128), LongestFirst()]


def make_plan(rng, windowed):
    needs = [CacheNeed(kv=KVNeed(2, 16, None))] * 2
    if windowed:
        needs = needs + [CacheNeed(kv=KVNeed(1, 16, 24))]      # a second group that gives pages back
    plan = CachePlan(needs, 400, 8, 16, False)
    caches = []
    for i in range(rng.randint(1, 12)):
        cache = plan.open(i)
        held = rng.randint(0, 90)
        plan.reserve(cache, held)
        plan.commit(cache, held)
        plan.reserve(cache, 1)
        caches.append(cache)
    return plan, caches


def packed_words(builder, packed):
    return builder._hosts[packed.turn].numpy()[:packed.layout.total].copy()


@pytest.mark.parametrize("seed", range(10))
def test_single_token_steps_pack_alike_both_ways(seed, monkeypatch):
    rng = random.Random(seed)
    plan, caches = make_plan(rng, windowed=seed % 2 == 1)
    entries = [StepEntry(c, [rng.randrange(1000)], rng.choice([[0], [], [0, 0]])) for c in caches]
    pads = {} if seed % 3 == 0 else dict(
        pad_requests=16, pad_tokens=16, pad_want=32,
        table_widths=[max(16, max(len(c.tables[g]) for c in caches)) for g in range(len(plan.groups))])
    outcomes = []
    for fast in (True, False):
        monkeypatch.setattr(batch_module, "_SINGLE_TOKEN_PATH", fast)
        builder = BatchBuilder(plan, 1000, 4096, torch.device("cpu"), NOTES)
        builder.validate(entries)
        packed = builder.pack(entries, **pads)
        outcomes.append((packed, packed_words(builder, packed)))
    (a, words_a), (b, words_b) = outcomes
    assert np.array_equal(words_a, words_b)
    for field in ("widths", "tokens", "requests", "wanted", "n_want", "q_lens", "kv_lens", "state_slots",
                  "note_counts"):
        assert getattr(a, field) == getattr(b, field), field
    assert a.layout == b.layout
    # what the annotations wrote: one tile of one row a request, most keys first; the order of
    # the third annotation, which the builder has never heard of
    lay, R = a.layout, len(entries)
    lengths = np.array([c.length + 1 for c in caches])
    tiles = words_a[lay.notes[0]:lay.notes[0] + 2 * R].reshape(R, 2)
    assert tiles[:, 1].tolist() == [1] * R and sorted(tiles[:, 0].tolist()) == list(range(R))
    assert (np.diff(lengths[tiles[:, 0]]) <= 0).all()
    assert words_a[lay.notes[2]:lay.notes[2] + R].tolist() == np.argsort(-lengths, kind="stable").tolist()
    assert a.note_counts[2] == R and a.note_counts[0] == (lay.note_words[0] // 2 if pads else R)


def test_what_a_step_may_not_bring():
    rng = random.Random(1)
    plan, caches = make_plan(rng, windowed=False)
    builder = BatchBuilder(plan, 1000, 4096, torch.device("cpu"))
    good = StepEntry(caches[0], [5], [0])
    builder.validate([good])
    for bad, text in ((StepEntry(caches[0], [], []), "brings no tokens"),
                      (StepEntry(caches[0], [1000], [0]), "outside the vocabulary"),
                      (StepEntry(caches[0], [-1], [0]), "outside the vocabulary"),
                      (StepEntry(caches[0], [3, 1000], [0]), "outside the vocabulary"),
                      (StepEntry(caches[0], [5], [1]), "wanted place"),
                      (StepEntry(caches[0], list(range(40)), [0]), "no pages reserved")):
        with pytest.raises(ValueError, match=text):
            builder.validate([bad])
    with pytest.raises(ValueError, match="appears twice"):
        builder.validate([good, StepEntry(caches[0], [6], [0])])
    plan.close(caches[0])
    with pytest.raises(ValueError, match="is closed"):
        builder.validate([good])

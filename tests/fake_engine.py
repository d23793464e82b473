"""A stand-in for the engine in scheduler tests: the real host-side cache plan,
and logits that are a fixed function of the request's whole history, so any
fault in cutting, preemption or recompute changes the sampled ids."""
import hashlib

import numpy as np

import plain_qwen2 as plain
from tokenizer_b200.cache import CachePlan
from tokenizer_b200.parts.base import CacheNeed, KVNeed


def logits_of(history, vocab):
    digest = hashlib.sha256(np.asarray(history, dtype=np.int64).tobytes()).digest()
    rng = np.random.RandomState(int.from_bytes(digest[:4], "little"))
    return rng.standard_normal(vocab).astype(np.float32) * 3.0


class FakeEngine:
    def __init__(self, num_pages, page_size=4, max_requests=8, vocab=50, max_positions=512,
                 share_prefixes=False, needs=None):
        needs = needs or [CacheNeed(kv=KVNeed(1, 8, None))]
        self.cache = CachePlan(needs, num_pages, page_size, max_requests, share_prefixes)
        self.vocab = vocab
        self.max_positions = max_positions
        self.page_contents = {}      # (page, offset) -> (token, position, digest of the prefix)
        self.history = {}            # id(cache) -> tokens the cache holds
        self.steps = []              # [(request id, n tokens)] per step

    def step(self, entries):
        rows = []
        self.steps.append([(e.cache.request_id, len(e.tokens)) for e in entries])
        for e in entries:
            assert len(e.tokens) > 0
            assert self.cache.pages_missing(e.cache, len(e.tokens)) == [0] * len(self.cache.groups)
            held = self.history.get(id(e.cache), [])
            if len(held) != e.cache.length:
                # pages adopted from a shared prefix: rebuild what they hold
                held = self._read_back(e.cache)
            assert len(held) == e.cache.length
            for i, token in enumerate(e.tokens):
                position = e.cache.length + i
                page = e.cache.tables[0][position // self.cache.page_size]
                assert page >= 0
                self.page_contents[(page, position % self.cache.page_size)] = (token, position)
                held = held + [token]
                if i in e.want:
                    rows.append(logits_of(held, self.vocab))
            self.history[id(e.cache)] = held
            self.cache.commit(e.cache, len(e.tokens))
        return np.stack(rows) if rows else np.zeros((0, self.vocab), dtype=np.float32)

    def decode_steps(self, entries, n_steps):
        """Greedy steps without the scheduler in between, as the engine offers them:
        pages for all the steps are reserved first, or nothing happens."""
        from tokenizer_b200.cache.manager import OutOfPages
        from tokenizer_b200.engine.batch import StepEntry
        missing = [0] * len(self.cache.groups)
        for e in entries:
            missing = [a + b for a, b in zip(missing, self.cache.pages_missing(e.cache, n_steps))]
        if any(m > a.available for m, a in zip(missing, self.cache.allocators)):
            raise OutOfPages("no pages for the burst")
        for e in entries:
            self.cache.reserve(e.cache, n_steps)
        self.bursts = getattr(self, "bursts", 0) + 1
        tokens = [e.tokens[0] for e in entries]
        out = []
        for _ in range(n_steps):
            logits = self.step([StepEntry(e.cache, [t], [0]) for e, t in zip(entries, tokens)])
            tokens = [int(np.argmax(row)) for row in logits]
            out.append(tokens)
        return out

    # ---- the engine's faces for a step packed ahead of its tokens (used when `ahead` is set) ----
    def enable_ahead(self, launch=False):
        """`launch`: the engine also runs a packed step with the ids of a draw that the host
        has not read yet."""
        self.prepared_used = 0
        self.launched_ahead = 0
        self.prepare_decode = self._prepare_decode
        self.step_prepared = self._step_prepared
        self.sample_launch = self._sample_launch
        if launch:
            self.step_prepared_device = self._step_prepared_device

    def _step_prepared_device(self, prepared, pending):
        assert not pending.read, "the step is launched before the host reads the draw"
        logits = self._step_prepared(prepared, pending.device_ids)
        if logits is not None:
            self.launched_ahead += 1
        return logits

    def _prepare_decode(self, caches):
        assert all(self.cache.pages_missing(c, 1) == [0] * len(self.cache.groups) for c in caches)
        return (list(caches), [c.length for c in caches])

    def _step_prepared(self, prepared, tokens):
        from tokenizer_b200.engine.batch import StepEntry
        caches, lengths = prepared
        if any(c.closed or c.length != n for c, n in zip(caches, lengths)) or len(tokens) != len(caches):
            return None
        self.prepared_used += 1
        return self.step([StepEntry(c, [t], [0]) for c, t in zip(caches, tokens)])

    def _sample_launch(self, logits, temperature, top_p, uniform):
        ids = self.sample(logits, temperature, top_p, uniform)

        class Pending:
            device_ids = ids
            read = False

            def result(self):
                self.read = True
                return ids
        return Pending()

    def _read_back(self, cache):
        out = []
        for position in range(cache.length):
            page = cache.tables[0][position // self.cache.page_size]
            token, at = self.page_contents[(page, position % self.cache.page_size)]
            assert at == position
            out.append(token)
        return out

    def sample(self, logits, temperature, top_p, uniform):
        return [plain.sample_token(row, t, p, u)
                for row, t, p, u in zip(np.asarray(logits), temperature, top_p, uniform)]

"""Continuous batching above the step function.

Every request is a *context* (its prompt and the ids sampled so far) and a
count of how much of that context the cache already holds.  One iteration:

 1. admit waiting requests in arrival order while a batch slot is free and the
    pool could hold the head's whole context now; a blocked head blocks those
    behind it, and a context that no empty pool could hold fails;
 2. give every running request its share of this step: requests one token short
    of their context (decoding) first, one token each, then the others get
    portions of their context, oldest first, under what is left of the token
    budget;
 3. reserve pages for those tokens, oldest request first.  When pages run out,
    the newest running request loses all its pages and goes back to the front
    of the waiting line; its context is run again later (nothing is sampled
    twice: a draw happens only when the whole context is in the cache).  A
    request that is alone and still does not fit fails;
 4. run the step, draw one id for each request whose context is now whole, let
    its cursor decide between going on and finishing, free what finished.

While the device draws the ids of a step in which every running request decodes, the
scheduler already reserves and packs the next step (`engine.prepare_decode`), and where the
engine can feed a step with drawn ids on the device (`engine.step_prepared_device`) it launches
that step before it has read the ids.  The next iteration then starts at 4 with the logits of
the step in flight; the rows of requests that ended with the ids read in between are dropped.

With `decode_burst` > 1 an iteration in which nobody waits, every running
request is decoding and draws greedily runs up to that many steps on the
device in one go (`engine.decode_steps`: each step's drawn ids are the next
step's inputs without a visit to the host) and then hands the ids to the
cursors one by one; ids after a request's end are dropped with its cache.  The
host's share of a step is paid once a burst.  When the pool has no pages for the
whole burst the iteration runs a single step as above.

The reference's scheduler (qwen-server/src/engine.rs:229-402, 455-704) admits
and preempts in the same way but runs a whole prompt per iteration; the token
budget and the portions are this engine's.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence

from ..cache.manager import OutOfPages
from .batch import StepEntry
from .generate import Control, Generated, GenerateParams, SampleCursor, StopReason


@dataclass
class SchedulerStats:
    steps: int = 0
    max_running: int = 0
    preemptions: int = 0
    last_preempted_id: int = -1
    requests_finished: int = 0
    requests_failed: int = 0
    peak_pages: int = 0
    tokens_run: int = 0
    tokens_sampled: int = 0
    shared_prefix_tokens: int = 0


@dataclass
class _Request:
    id: int
    prompt: List[int]
    cursor: SampleCursor
    context: List[int]
    cache: object = None
    published: bool = False
    arrived: float = 0.0
    prompt_done: Optional[float] = None


class Scheduler:
    def __init__(self, engine, max_batch_size: int = 8, token_budget: int = 512,
                 decode_burst: int = 1):
        """`engine` offers `cache` (a CachePlan), `step(entries) -> logits`,
        `sample(logits, temperature, top_p, uniform) -> ids` and
        `max_positions`; for bursts also `decode_steps(entries, n) -> ids[n][entries]`."""
        if max_batch_size < 1 or token_budget < 1:
            raise ValueError("the batch holds at least one request and one token")
        if decode_burst < 1:
            raise ValueError("a burst is at least one step")
        self.decode_burst = decode_burst if hasattr(engine, "decode_steps") else 1
        self.engine = engine
        self.cache = engine.cache
        if max_batch_size > self.cache.max_requests:
            raise ValueError(f"a batch of {max_batch_size} requests needs as many request slots; "
                             f"the cache has {self.cache.max_requests}")
        self.max_batch_size = max_batch_size
        self.token_budget = token_budget
        self.waiting: Deque[_Request] = deque()
        self.running: List[_Request] = []
        self.finished: Dict[int, Generated] = {}
        self.stats = SchedulerStats()
        self._next_id = 0
        self._ahead = None            # (requests, step packed ahead of its tokens)
        self._in_flight = None        # (requests, logits) of a step launched ahead of its tokens

    # ---- requests -------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: GenerateParams,
                    token_bytes: Optional[Callable[[int], bytes]] = None,
                    on_chunk: Optional[Callable[[str], Control]] = None) -> int:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("the prompt has no tokens")
        if len(prompt) + params.max_tokens > self.engine.max_positions:
            raise ValueError(
                f"prompt of {len(prompt)} plus max_tokens {params.max_tokens} exceeds "
                f"max_position_embeddings {self.engine.max_positions}")
        request = _Request(self._next_id, prompt, SampleCursor(params, token_bytes, on_chunk),
                           list(prompt), arrived=time.perf_counter())
        self._next_id += 1
        self.waiting.append(request)
        return request.id

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def run(self) -> Dict[int, Generated]:
        while self.has_work():
            self.step()
        return self.finished

    # ---- one iteration -----------------------------------------------------------
    def step(self) -> List[int]:
        """Run one iteration; returns the ids of the requests that finished."""
        done_before = set(self.finished)
        self._admit()
        in_flight, self._in_flight = self._in_flight, None
        if in_flight is not None:
            # this step already runs (or ran) on the device, fed with the last draw's ids there;
            # what it computed for requests that ended with those ids is dropped
            requests, logits = in_flight
            alive = [i for i, r in enumerate(requests) if r.cursor.done is None]
            if alive:
                self._sample([requests[i] for i in alive],
                             logits if len(alive) == len(requests) else logits[alive])
                return [i for i in self.finished if i not in done_before]
        ahead, self._ahead = self._ahead, None
        burst = self._burst_length()
        if burst > 1 and self._run_burst(burst):
            return [i for i in self.finished if i not in done_before]
        plan, logits = None, None
        if ahead is not None and self._still_holds(ahead[0]):
            # the step was packed while the last one ran: only the tokens were missing
            logits = self.engine.step_prepared(ahead[1], [r.context[-1] for r in ahead[0]])
            if logits is not None:
                plan = [(r, 1) for r in ahead[0]]
        if logits is None:
            plan = self._plan_and_reserve()
            if plan:
                entries = [StepEntry(r.cache, r.context[r.cache.length:r.cache.length + n],
                                     [n - 1] if r.cache.length + n == len(r.context) else [])
                           for r, n in plan]
                logits = self.engine.step(entries)
        if plan:
            for r, n in plan:
                # whole pages of a prompt are offered to later requests as soon as they are
                # computed, not only when the prompt is complete (a long prompt runs over
                # several steps, and requests behind it may begin with the same tokens)
                if not r.published and n > 1 and r.cache.length < len(r.prompt):
                    self.cache.publish_prompt(r.cache, r.prompt[:r.cache.length])
            self.stats.steps += 1
            self.stats.tokens_run += sum(n for _, n in plan)
            self.stats.max_running = max(self.stats.max_running, len(self.running))
            self.stats.peak_pages = max(
                self.stats.peak_pages, max((a.live for a in self.cache.allocators), default=0))
            self._sample([r for r, n in plan if r.cache.length == len(r.context)], logits)
        return [i for i in self.finished if i not in done_before]

    def _still_holds(self, requests) -> bool:
        """A step packed ahead is good if exactly these requests run, nobody waits, and each
        is one token short of its context."""
        if self.waiting or len(requests) != len(self.running):
            return False
        running = sorted(self.running, key=lambda r: r.id)
        return all(a is b and a.cursor.done is None and len(a.context) - a.cache.length == 1
                   for a, b in zip(running, requests))

    def _pack_ahead(self, ready: List[_Request]) -> None:
        """While the device still draws this step's ids: if the next step will be one token
        for each of the requests that run now, reserve its pages and let the engine pack it.
        Should a request end with the id it is about to get, the packed step is dropped."""
        prepare = getattr(self.engine, "prepare_decode", None)
        if prepare is None or self.waiting or len(ready) != len(self.running) or self.decode_burst > 1:
            return
        if any(r.cursor.produced + 1 >= r.cursor.params.max_tokens or
               len(r.context) + 1 >= self.engine.max_positions for r in ready):
            return
        requests = sorted(ready, key=lambda r: r.id)
        try:
            for r in requests:
                self.cache.reserve(r.cache, 1)
        except OutOfPages:
            return                       # the next iteration decides who gives way
        prepared = prepare([r.cache for r in requests])
        if prepared is not None:
            self._ahead = (requests, prepared)

    def _launch_ahead(self, drawing: List[_Request], pending) -> None:
        """If the next step is packed and the engine can take its tokens from the draw on the
        device, launch it now: the host reads the drawn ids, extends the contexts and judges
        the ends while that step runs, instead of the device waiting for the host.  A request
        that ends with the id being drawn (an end-of-sequence id, a stop text, a callback; never
        `max_tokens`, which `_pack_ahead` sees coming) has then run one token that nobody reads."""
        run = getattr(self.engine, "step_prepared_device", None)
        if run is None or self._ahead is None:
            return
        requests, prepared = self._ahead
        if len(requests) != len(drawing) or any(a is not b for a, b in zip(requests, drawing)):
            return                        # the draw's rows are in another order than the packed step's
        logits = run(prepared, pending)
        if logits is None:
            return
        self._ahead = None
        self._in_flight = (requests, logits)
        self.stats.steps += 1
        self.stats.tokens_run += len(requests)

    def _burst_length(self) -> int:
        """How many steps the running requests can take together on the device:
        0 unless nobody waits and all of them decode greedily."""
        if self.decode_burst <= 1 or self.waiting or not self.running:
            return 0
        n = self.decode_burst
        for r in self.running:
            c = r.cursor
            if len(r.context) - r.cache.length != 1 or c.params.temperature != 0.0 or c.done is not None:
                return 0
            n = min(n, c.params.max_tokens - c.produced, self.engine.max_positions - len(r.context))
        return n

    def _run_burst(self, n: int) -> bool:
        ready = sorted(self.running, key=lambda r: r.id)
        entries = [StepEntry(r.cache, [r.context[-1]]) for r in ready]
        try:
            ids = self.engine.decode_steps(entries, n)
        except OutOfPages:
            return False                  # nothing was reserved or run: take a single step
        self.stats.steps += n
        self.stats.tokens_run += n * len(ready)
        self.stats.max_running = max(self.stats.max_running, len(self.running))
        self.stats.peak_pages = max(
            self.stats.peak_pages, max((a.live for a in self.cache.allocators), default=0))
        now = time.perf_counter()
        for at, r in enumerate(ready):
            for k in range(n):
                self.stats.tokens_sampled += 1
                token = int(ids[k][at])
                if not r.cursor.accept(token):
                    break
                r.context.append(token)
            if r.cursor.done is not None:
                self._retire(r, now)
        return True

    def _context_pages(self, request: _Request) -> int:
        return self.cache.pages_for_tokens(len(request.context))

    def _admit(self) -> None:
        while self.waiting and len(self.running) < self.max_batch_size:
            head = self.waiting[0]
            if self._context_pages(head) > self.cache.num_pages:
                self.waiting.popleft()
                self._fail(head, f"the cache has {self.cache.num_pages} pages of "
                                 f"{self.cache.page_size}; this request needs {self._context_pages(head)}")
                continue
            try:
                cache = self.cache.open(head.id)
            except OutOfPages:
                break                    # every request slot is held (some outside this scheduler): wait
            adopted = self.cache.adopt_prefix(cache, head.context[:-1])
            if not self.cache.can_reserve(cache, len(head.context) - cache.length):
                self.cache.close(cache)
                break
            self.stats.shared_prefix_tokens += adopted
            head.cache = cache
            self.running.append(self.waiting.popleft())

    def _adopt_late(self, r: _Request) -> None:
        """A running request that holds nothing yet looks once more for pages that hold the
        beginning of its context: requests admitted in the same iteration as the one that
        computes a shared beginning find nothing at admission, but by the time their first
        portion gets a share of a step, those pages have been published."""
        if r.cache.length == 0 and not any(r.cache.tables):
            self.stats.shared_prefix_tokens += self.cache.adopt_prefix(r.cache, r.context[:-1])

    def _shares(self) -> List:
        """(request, tokens this step): decoding requests first, then portions
        of contexts, oldest first, under the token budget."""
        by_age = sorted(self.running, key=lambda r: r.id)
        left = self.token_budget
        shares = []
        for r in by_age:
            if len(r.context) - r.cache.length == 1:
                shares.append((r, 1))
                left -= 1
        for r in by_age:
            if left > 0 and len(r.context) - r.cache.length > 1:
                self._adopt_late(r)
            remaining = len(r.context) - r.cache.length
            if remaining > 1 and left > 0:
                shares.append((r, min(remaining, left)))
                left -= shares[-1][1]
            elif remaining == 1 and left > 0 and all(r is not s[0] for s in shares):
                shares.append((r, 1))          # all but its last token were taken over just now
                left -= 1
        return shares

    def _plan_and_reserve(self) -> List:
        while True:
            shares = self._shares()
            short = None
            for r, n in sorted(shares, key=lambda s: s[0].id):
                try:
                    self.cache.reserve(r.cache, n)
                except OutOfPages:
                    short = r
                    break
            if short is None:
                return shares
            victim = max(self.running, key=lambda r: r.id)
            if victim is short and len(self.running) == 1:
                self.running.remove(short)
                self.cache.close(short.cache)
                self._fail(short, f"the cache has {self.cache.num_pages} pages of "
                                  f"{self.cache.page_size}; this request cannot go on alone")
                continue
            self._preempt(victim)

    def _preempt(self, victim: _Request) -> None:
        self.running.remove(victim)
        self.cache.close(victim.cache)
        victim.cache = None
        self.stats.preemptions += 1
        self.stats.last_preempted_id = victim.id
        # To the front of the line.  Victims are taken newest first and every
        # waiting request is newer than any running one, so the line stays in
        # arrival order.
        self.waiting.appendleft(victim)

    def _sample(self, ready: List[_Request], logits) -> None:
        now = time.perf_counter()
        rows, drawing = [], []
        for row, r in enumerate(ready):
            if r.prompt_done is None:
                r.prompt_done = now
            if not r.published and r.cache.length >= len(r.prompt):
                self.cache.publish_prompt(r.cache, r.prompt)
                r.published = True
            if r.cursor.wants_sample():
                rows.append(row)
                drawing.append(r)
        if drawing:
            picked = logits if len(rows) == len(ready) else logits[rows]
            draw = [picked, [r.cursor.params.temperature for r in drawing],
                    [r.cursor.params.top_p for r in drawing],
                    [r.cursor.next_uniform() for r in drawing]]
            launch = getattr(self.engine, "sample_launch", None)
            if launch is None:
                ids = self.engine.sample(*draw)
            else:
                pending = launch(*draw)
                if len(drawing) == len(ready):
                    self._pack_ahead(ready)          # beside the device
                    self._launch_ahead(drawing, pending)
                ids = pending.result()
            self.stats.tokens_sampled += len(ids)
            for r, token in zip(drawing, ids):
                if r.cursor.accept(int(token)):
                    r.context.append(int(token))
        for r in ready:
            if r.cursor.done is not None:
                self._retire(r, now)

    def _retire(self, r: _Request, now: float) -> None:
        self.running.remove(r)
        self.cache.close(r.cache)
        r.cache = None
        result = r.cursor.done
        result.prefill = (r.prompt_done or now) - r.arrived
        result.decode = time.perf_counter() - (r.prompt_done or now)
        self.finished[r.id] = result
        self.stats.requests_finished += 1

    def _fail(self, r: _Request, message: str) -> None:
        self.finished[r.id] = Generated(list(r.cursor.tokens), r.cursor.text, list(r.cursor.chunks),
                                        StopReason.FAILED, r.cursor.produced, error=message)
        self.stats.requests_failed += 1

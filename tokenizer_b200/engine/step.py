"""The engine and its one step function.

`Engine.step(entries)` runs a batch of (request, its next tokens): portions of
prompts beside single decoded tokens, cut anywhere.  It runs only the tokens it
is given, as one batch, against the cache that earlier steps left, writes their
keys and values into the pages reserved for them, and returns the float32
logits at the wanted places.  Pages are reserved by the caller (the scheduler
or the replay program) through `engine.cache`; the step itself allocates none,
as the reference's paged forwards do not (qwen-infer/src/model.rs:1015-1053).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..cache.device import DeviceCache
from ..config.registry import load_config
from ..kernels import ops
from ..kernels.ops import KernelError
from ..parts.base import Runtime
from ..parts.model import DecoderModel
from ..weights.store import WeightStore
from ..sampling.sampler import Sampler
from .batch import BatchBuilder, StepEntry

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _DTYPES[str(name)]
    except KeyError:
        raise ValueError(f"dtype is bfloat16 or float32, found {name!r}") from None


def load_model(folder: str, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """Build the model that the folder's config.json names, with the folder's
    weights, on `device`.  There is no CPU path."""
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise KernelError(
            "tokenizer_b200 runs on a CUDA GPU (sm_100a) only; no GPU is visible to this process")
    config = load_config(folder)
    store = WeightStore.from_folder(folder)
    with torch.cuda.device(device):
        model = DecoderModel(config.model_spec(), store, Runtime(device, parse_dtype(dtype)))
    model.config = config
    return model


def random_model(config, seed: int, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """The model of a typed configuration with seeded random weights drawn on the device, no
    folder in between (for sizes whose file would be many gigabytes).  Same parts, same checks
    as `load_model`; the values are not those of `write_random_model` for the same seed."""
    from ..parts.model import declared_tensors
    from ..weights import SeededTensors
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise KernelError(
            "tokenizer_b200 runs on a CUDA GPU (sm_100a) only; no GPU is visible to this process")
    spec = config.model_spec()
    store = WeightStore(SeededTensors(declared_tensors(spec), seed, device), "<seeded random weights>")
    with torch.cuda.device(device):
        model = DecoderModel(spec, store, Runtime(device, parse_dtype(dtype)))
    model.config = config
    return model


class PreparedDecode:
    """A decoding step whose metadata is packed and whose tokens are still to come."""

    def __init__(self, entries, key, packed, lengths):
        self.entries, self.key, self.packed, self.lengths = entries, key, packed, lengths


class Engine:
    def __init__(self, model: DecoderModel, num_pages: int, page_size: int = 16,
                 max_requests: int = 64, share_prefixes: bool = False, use_graphs: bool = True):
        self.model = model
        self.runtime = model.runtime
        self.cache = DeviceCache(model.cache_needs(), num_pages, page_size, max_requests,
                                 model.runtime, share_prefixes)
        self.bindings = self.cache.bindings(model.order)
        self.builder = BatchBuilder(self.cache, model.vocab_size, model.max_positions,
                                    model.runtime.device, model.batch_annotations())
        self.sampler = Sampler(model.runtime.device)
        self.max_positions = model.max_positions
        self.steps_run = 0
        self.steps_fed_on_device = 0      # of them: launched with a draw's ids before the host read them
        # a captured step bakes its launches: only mixers that say so may be replayed, and a
        # feed-forward may say that it cannot (a choice made on the host, say)
        self.use_graphs = bool(use_graphs) and model.graph_safe()
        self._graphs = {}
        self._graph_buffer = 0
        tables = sum(max_requests * (model.max_positions // page_size + 8) for _ in self.cache.groups)
        self.builder.reserve_capacity(16 * 8192 + tables)

    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0", **kw) -> "Engine":
        return cls(load_model(folder, dtype, device), **kw)

    def check(self) -> None:
        """Raise `KernelError` if a bounded wait inside a kernel ran out since the last check
        (the kernel then ran on without its data and what the steps since wrote is wrong).
        It reads one word of host memory; it is meaningful for the work the host has already
        waited for, so callers that read logits or ids themselves call it after that read.
        `step`, `decode_steps`, the prepared steps and the sampler's `result()` call it."""
        ops.raise_if_error()

    def step(self, entries: List[StepEntry]) -> torch.Tensor:
        """Run one batch; returns logits [wanted, vocab] float32 on the device,
        in the order of the entries and of their `want`.

        The logits are valid until the engine's next step: a step replayed from a captured
        graph returns a view of that graph's output buffer, which the next replay of the same
        shape overwrites.  A caller that keeps logits across steps clones them."""
        self.check()
        if not entries:
            return torch.empty((0, self.model.vocab_size), dtype=torch.float32,
                               device=self.runtime.device)
        self.builder.validate(entries)
        with torch.cuda.device(self.runtime.device):
            shape = self._captured_shape(entries) if self.use_graphs else None
            if shape is not None:
                logits = self._step_captured(entries, *shape)
            else:
                ctx, want_rows, n_want = self.builder.build(entries)
                logits = self.model.forward(ctx, self.bindings, want_rows[:n_want])
        for e in entries:
            self.cache.commit(e.cache, len(e.tokens))
        self.steps_run += 1
        return logits

    # ---- decoding steps replayed from CUDA graphs ---------------------------------
    @staticmethod
    def _width(pages: int) -> int:
        """Captured block-table widths: powers of two up to 64 pages, then whole 64s (kernels
        size their grids from the table's reach, so a width twice the need costs idle blocks)."""
        if pages <= 64:
            return Engine._bucket(pages, 8)
        return -(-pages // 64) * 64

    @staticmethod
    def _bucket(n: int, least: int = 1) -> int:
        b = least
        while b < n:
            b *= 2
        return b

    # captured shapes of prompt steps are kept while their tokens add up to at most this (each
    # holds its own activations, which grow with its tokens: a 2,048-token shape of a small
    # model some hundred megabytes, a 512-token shape a quarter of that)
    PORTION_GRAPH_TOKENS = 24576

    def _captured_shape(self, entries: List[StepEntry]):
        """(key, padded tokens, padded requests) when steps of this shape are replayed
        from a captured graph, else None.  Steps of single tokens always are.  Steps
        with prompt portions are when they bring (nearly) a whole number of 128-token tiles
        or fewer than 256 tokens: under a token budget most steps of a busy engine bring exactly
        the budget, and a replay spares the host the launches (a quarter of such a step's
        time otherwise, two thirds of a short step's).  What the model's parts say decides their kernels beyond the
        sizes (`shape_key`) is part of the key."""
        pages = [max(len(e.cache.tables[g]) for e in entries) for g in range(len(self.cache.groups))]
        longest = max(len(e.tokens) for e in entries)
        if longest == 1:
            rows = self._bucket(len(entries))
            return (rows, tuple(self._width(n) for n in pages)), rows, rows
        # the kernels for portions size their grids from the rows, not from the tables' reach:
        # powers of two keep the shapes of a busy scheduler few
        widths = tuple(self._bucket(n, 8) for n in pages)
        total = sum(len(e.tokens) for e in entries)
        requests = self._bucket(len(entries))
        # up to the next whole tile with idle rows, where that wastes little (a sixteenth); a short
        # step (a short prompt, the last portion of a long one) is padded to whole half tiles (to 16
        # rows under 64) whatever that wastes: launched from the host its 200 launches take 3 ms, replayed a third of that
        if total >= 256:
            padded = -(-total // 128) * 128
            if padded - total > total // 16:
                return None
        elif total >= 64:
            padded = -(-total // 64) * 64
        else:
            padded = -(-total // 16) * 16
        if sum(len(e.want) for e in entries) > requests:
            return None
        kinds = self.model.shape_key([len(e.tokens) for e in entries])
        return ("portions", padded, requests, widths, kinds), padded, requests

    def _step_captured(self, entries: List[StepEntry], key, tokens: int, requests: int) -> torch.Tensor:
        """A step whose launches are captured once per shape (padded batch size,
        padded block-table widths, token count) and replayed afterwards; only the
        packed metadata changes between replays, at fixed addresses.  Idle rows of
        the padded batch carry request -1, which kernels skip."""
        from ..kernels.ops import counter
        widths = list(key[1] if len(key) == 2 else key[3])
        ctx, want_rows, n_want = self.builder.build(
            entries, pad_requests=requests, pad_tokens=tokens, pad_want=requests, table_widths=widths)
        if self._graph_buffer != self.builder.device_buffer_ptr():
            self._graphs.clear()           # the metadata moved: captured addresses are stale
            self._graph_buffer = self.builder.device_buffer_ptr()
        slot = self._graphs.get(key)
        if slot is None:
            # first use: run it once plainly (this also compiles what is missing)
            if key[0] == "portions":
                kept = [k for k in self._graphs if k[0] == "portions"]
                while kept and sum(k[1] for k in kept) + key[1] > self.PORTION_GRAPH_TOKENS:
                    del self._graphs[kept.pop(0)]      # the oldest shapes make room
            self._graphs[key] = {}
            return self.model.forward(ctx, self.bindings, want_rows)[:n_want]
        if "graph" not in slot:
            graph = torch.cuda.CUDAGraph()
            before = counter.launches
            torch.cuda.synchronize()
            with torch.cuda.graph(graph):
                out = self.model.forward(ctx, self.bindings, want_rows)
            slot.update(graph=graph, out=out, launches=counter.launches - before)
            counter.launches = before
        slot["graph"].replay()
        counter.launches += slot["launches"]
        return slot["out"][:n_want]

    def decode_steps(self, entries: List[StepEntry], n_steps: int) -> List[List[int]]:
        """Greedy decoding of `n_steps` tokens for every entry without going
        back to the host between steps: each entry brings the one token to run
        next; the drawn id becomes the next input on the device.  Returns the
        drawn ids, [n_steps][len(entries)].  Pages for all the steps are
        reserved here; OutOfPages leaves everything as it was."""
        from ..kernels import ops
        from ..kernels.ops import counter
        if n_steps <= 0 or not entries:
            return []
        for e in entries:
            if len(e.tokens) != 1:
                raise ValueError("decode_steps takes one token per request")
            if e.cache.length + n_steps > self.max_positions:
                raise ValueError("the steps would pass max_position_embeddings")
        for e in entries:
            if not self.cache.can_reserve(e.cache, n_steps):
                from ..cache.manager import OutOfPages
                raise OutOfPages(f"no pages for {n_steps} more tokens of {e.cache.request_id!r}")
        for e in entries:
            self.cache.reserve(e.cache, n_steps)
        for e in entries:
            e.want = [0]
        self.builder.validate(entries)
        device = self.runtime.device
        with torch.cuda.device(device):
            rows = self._bucket(len(entries))
            widths = [self._width(max(len(e.cache.tables[g]) for e in entries))
                      for g in range(len(self.cache.groups))]
            ctx, want_rows, n_want = self.builder.build(
                entries, pad_requests=rows, pad_tokens=rows, pad_want=rows, table_widths=widths)
            if self._graph_buffer != self.builder.device_buffer_ptr():
                self._graphs.clear()
                self._graph_buffer = self.builder.device_buffer_ptr()
            key = ("steps", rows, tuple(widths))
            slot = self._graphs.get(key)
            if slot is None:
                slot = self._graphs[key] = {
                    "history": torch.zeros(4096 * rows, dtype=torch.int32, device=device),
                    "counter": torch.zeros(1, dtype=torch.int32, device=device),
                    "drawn": torch.zeros(rows, dtype=torch.int32, device=device)}
            if n_steps > 4096:
                raise ValueError("decode_steps runs at most 4096 steps a call")
            slot["counter"].zero_()

            def iteration():
                logits = self.model.forward(ctx, self.bindings, want_rows)
                with ops.scratch_scope(self.sampler.scratch):
                    ops.sample(logits, None, None, None, slot["drawn"])
                ops.advance_decode(ctx.ids, slot["drawn"], ctx.pos, ctx.kv_len, ctx.row_req,
                                   [g.slots for g in ctx.groups],
                                   [g.block_table for g in ctx.groups], self.cache.page_size,
                                   slot["history"], slot["counter"])
                # a mixer that keeps more than keys and values between steps moves it on here
                for call, binding in zip(self.model.order, self.bindings):
                    advance = getattr(self.model.blocks[call.layer].mixer, "advance_decode", None)
                    if advance is not None:
                        advance(ctx, binding)

            done = 0
            if not self.use_graphs:
                # a part whose launches depend on host-side values cannot be replayed: every
                # step is launched anew (still without a visit to the host for the ids)
                for _ in range(n_steps):
                    iteration()
                    ctx.kv_lens = [n + 1 for n in ctx.kv_lens]      # the host's copies follow
                done = n_steps
            elif "graph" not in slot:
                iteration()              # plainly once: compiles and warms
                done = 1
                if n_steps > 1:
                    graph = torch.cuda.CUDAGraph()
                    before = counter.launches
                    torch.cuda.synchronize()
                    # capture replays the step on the live metadata; it does not run
                    with torch.cuda.graph(graph):
                        iteration()
                    slot.update(graph=graph, launches=counter.launches - before)
                    counter.launches = before
            for _ in range(done, n_steps):
                slot["graph"].replay()
                counter.launches += slot["launches"]
            history = slot["history"][:n_steps * rows].view(n_steps, rows)[:, :len(entries)].tolist()
        self.check()
        for e in entries:
            self.cache.commit(e.cache, n_steps)
        self.steps_run += n_steps
        return history

    def sample(self, logits: torch.Tensor, temperature, top_p, uniform) -> List[int]:
        """Draw one id per row of `logits` on the device."""
        return self.sample_launch(logits, temperature, top_p, uniform).result()

    def sample_launch(self, logits: torch.Tensor, temperature, top_p, uniform):
        """Start the draw; `.result()` of what is returned waits for the ids."""
        with torch.cuda.device(self.runtime.device):
            return self.sampler.sample_launch(logits, temperature, top_p, uniform)

    # ---- a decoding step packed ahead of its tokens --------------------------------
    def prepare_decode(self, caches) -> Optional["PreparedDecode"]:
        """Pack, on the host only, a step that will run one token (not yet known) for each
        cache, wanting its logits; pages for the token must be reserved.  None when steps of
        this shape are not replayed from a graph yet.  The scheduler calls this while the
        device still runs the step before, so that the host's share of a step is hidden."""
        if not self.use_graphs or not caches:
            return None
        entries = [StepEntry(c, [0], [0]) for c in caches]
        key, tokens, requests = self._captured_shape(entries)
        slot = self._graphs.get(key)
        if slot is None or "graph" not in slot or self._graph_buffer != self.builder.device_buffer_ptr():
            return None
        self.builder.validate(entries)
        packed = self.builder.pack(entries, pad_requests=requests, pad_tokens=tokens,
                                   pad_want=requests, table_widths=list(key[1]))
        return PreparedDecode(entries, key, packed, [c.length for c in caches])

    def step_prepared_device(self, prepared: "PreparedDecode", pending) -> Optional[torch.Tensor]:
        """As `step_prepared`, with the tokens taken on the device from a draw that was launched
        (`sample_launch`) and not read yet: the step starts right behind the draw, and the host
        reads and judges the drawn ids while it runs.  A request that turns out to have ended
        with its drawn id has then run one token too many, which nobody reads.  None when the
        step cannot be used as packed."""
        from ..kernels.ops import counter
        self.check()
        ids = getattr(pending, "device_ids", None)
        slot = self._graphs.get(prepared.key)
        if ids is None or ids.numel() != len(prepared.entries) or ids.dtype != torch.int32 or \
                slot is None or "graph" not in slot or self._graph_buffer != self.builder.device_buffer_ptr() or \
                any(e.cache.closed or e.cache.length != n for e, n in zip(prepared.entries, prepared.lengths)):
            return None
        with torch.cuda.device(self.runtime.device):
            n_want = self.builder.copy(prepared.packed)
            self.builder.copy_ids(prepared.packed, ids)
            slot["graph"].replay()
            counter.launches += slot["launches"]
        for e in prepared.entries:
            self.cache.commit(e.cache, 1)
        self.steps_run += 1
        self.steps_fed_on_device += 1
        return slot["out"][:n_want]

    def step_prepared(self, prepared: "PreparedDecode", tokens: Sequence[int]) -> Optional[torch.Tensor]:
        """Run a step packed by `prepare_decode` with the tokens now known.  None when it can
        no longer be used as packed (a cache moved on, the graph is gone): run `step` instead."""
        from ..kernels.ops import counter
        self.check()
        slot = self._graphs.get(prepared.key)
        if slot is None or "graph" not in slot or self._graph_buffer != self.builder.device_buffer_ptr() or \
                len(tokens) != len(prepared.entries) or \
                any(e.cache.closed or e.cache.length != n for e, n in zip(prepared.entries, prepared.lengths)):
            return None
        for t in tokens:
            if not 0 <= int(t) < self.model.vocab_size:
                raise ValueError(f"token id {t} is outside the vocabulary of {self.model.vocab_size}")
        self.builder.set_ids(prepared.packed, tokens)
        with torch.cuda.device(self.runtime.device):
            n_want = self.builder.copy(prepared.packed)
            slot["graph"].replay()
            counter.launches += slot["launches"]
        for e in prepared.entries:
            self.cache.commit(e.cache, 1)
        self.steps_run += 1
        return slot["out"][:n_want]

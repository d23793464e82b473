"""Turning a step's entries into the device-side description of the batch.

All integer metadata of a step (ids, positions, the request of each row, cache
slots, block tables, wanted rows) is packed into ONE int32 buffer on the host
and copied to the device with one transfer; the parts receive views into it.
The layout is a function of the capacities alone, so a step replayed from a
captured graph finds every array at the same address.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import RequestCache
from ..parts.base import GroupView, StepContext


@dataclass
class StepEntry:
    """A request's share of one step: its next tokens and the places among
    them (0-based) whose logits are wanted."""

    cache: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()


def _round4(n: int) -> int:
    return (n + 3) // 4 * 4


@dataclass
class BatchLayout:
    """Offsets (in int32 elements) of every array in the packed buffer."""

    T: int
    R: int
    W: int
    table_widths: List[int]
    ids: int = 0
    pos: int = 0
    row_req: int = 0
    q_start: int = 0
    kv_len: int = 0
    state_slot: int = 0
    want: int = 0
    notes: Optional[List[int]] = None         # offsets of the parts' annotations ...
    note_words: Optional[List[int]] = None    # ... and their sizes
    slots: Optional[List[int]] = None
    tables: Optional[List[int]] = None
    total: int = 0

    @classmethod
    def compute(cls, T: int, R: int, W: int, table_widths: List[int], annotations=()) -> "BatchLayout":
        lay = cls(T, R, W, list(table_widths))
        at = 0

        def take(n):
            nonlocal at
            start = at
            at += _round4(max(n, 1))
            return start

        lay.ids, lay.pos, lay.row_req = take(T), take(T), take(T)
        lay.q_start, lay.kv_len, lay.state_slot = take(R + 1), take(R), take(R)
        lay.want = take(W)
        lay.note_words = [int(a.capacity(T, R)) for a in annotations]
        lay.notes = [take(n) for n in lay.note_words]
        lay.slots = [take(T) for _ in table_widths]
        lay.tables = [take(R * w) for w in table_widths]
        lay.total = at
        return lay


@dataclass
class PackedStep:
    """A step packed into one of the builder's pinned buffers, not yet copied."""

    layout: BatchLayout
    turn: int
    widths: List[int]
    tokens: int
    requests: int
    wanted: int
    n_want: int
    q_lens: List[int]
    kv_lens: List[int]
    state_slots: List[int]
    note_counts: List[int]            # what each annotation's `fill` returned


# False sends steps of single tokens through the general packing loop too (tests compare the two)
_SINGLE_TOKEN_PATH = True


class BatchBuilder:
    def __init__(self, plan, vocab_size: int, max_positions: int, device, annotations=()):
        """`annotations`: the `BatchAnnotation`s of the model's parts, one per key."""
        self.annotations = list(annotations)
        self.plan = plan
        self.vocab_size = vocab_size
        self.max_positions = max_positions
        self.device = device
        # two pinned buffers used in turn: the next step can be packed while the copy of
        # the one before may still be reading its buffer
        self._hosts: List[Optional[torch.Tensor]] = [None, None]
        self._copied: List[Optional[torch.cuda.Event]] = [None, None]
        self._turn = 0
        self._dev: Optional[torch.Tensor] = None
        self.last_bytes = 0

    def _buffers(self, total: int):
        if self._dev is None or self._dev.numel() < total:
            capacity = max(total * 2, 4096)
            pin = self.device.type == "cuda"
            self._hosts = [torch.empty(capacity, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
            self._copied = [None, None]
            self._dev = torch.empty(capacity, dtype=torch.int32, device=self.device)
        return self._dev

    def device_buffer_ptr(self) -> int:
        return 0 if self._dev is None else self._dev.data_ptr()

    def reserve_capacity(self, total: int) -> None:
        """Size the buffers once, so that later steps never move them (captured
        graphs hold their addresses)."""
        self._buffers(total)

    def validate(self, entries: List[StepEntry]) -> None:
        seen = set()
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.cache.request_id!r} brings no tokens to this step")
            if e.cache.closed:
                raise ValueError(f"request {e.cache.request_id!r} is closed")
            if id(e.cache) in seen:
                raise ValueError(f"request {e.cache.request_id!r} appears twice in one step")
            seen.add(id(e.cache))
            if e.cache.length + n > self.max_positions:
                raise ValueError(
                    f"positions {e.cache.length}..{e.cache.length + n} exceed "
                    f"max_position_embeddings {self.max_positions}")
            if n == 1:
                if not 0 <= int(e.tokens[0]) < self.vocab_size:
                    raise ValueError(f"token id {int(e.tokens[0])} is outside the vocabulary of {self.vocab_size}")
            else:
                ids = np.asarray(e.tokens, dtype=np.int64)
                if int(ids.min()) < 0 or int(ids.max()) >= self.vocab_size:
                    bad = int(ids[(ids < 0) | (ids >= self.vocab_size)][0])
                    raise ValueError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise ValueError(f"wanted place {w} is not among the {n} tokens brought")
            if any(self.plan.pages_missing(e.cache, n)):
                raise ValueError(
                    f"request {e.cache.request_id!r} has no pages reserved for {n} more tokens")

    def build(self, entries: List[StepEntry], pad_requests: int = 0, pad_tokens: int = 0,
              pad_want: int = 0, table_widths: Optional[List[int]] = None):
        """Pack the step.  The `pad_*` capacities (graph replay) extend the
        batch with idle rows: request index -1, which every kernel skips.  A padded
        step also announces the most tiles its shape can have (the unused ones have
        no rows), so that a captured launch fits every step of the shape."""
        return self.upload(self.pack(entries, pad_requests, pad_tokens, pad_want, table_widths))

    def pack(self, entries: List[StepEntry], pad_requests: int = 0, pad_tokens: int = 0,
             pad_want: int = 0, table_widths: Optional[List[int]] = None) -> "PackedStep":
        """The host's half of `build`: fill a pinned buffer; nothing touches the device."""
        padded = bool(pad_requests or pad_tokens or pad_want or table_widths)
        plan = self.plan
        page = plan.page_size
        T = sum(len(e.tokens) for e in entries)
        R = len(entries)
        W = sum(len(e.want) for e in entries)
        widths = []
        for g in range(len(plan.groups)):
            need = max([len(e.cache.tables[g]) for e in entries] + [1])
            widths.append(need if table_widths is None else table_widths[g])
            if widths[-1] < need:
                raise ValueError("the captured block-table width is too small for this step")
        Tc, Rc, Wc = max(T, pad_tokens), max(R, pad_requests), max(W, pad_want)
        lay = BatchLayout.compute(Tc, Rc, Wc, widths, self.annotations)
        self._buffers(lay.total)
        turn = self._turn
        self._turn ^= 1
        if self._copied[turn] is not None:
            self._copied[turn].synchronize()  # the copy of two steps ago still reads this buffer
            self._copied[turn] = None
        buf = self._hosts[turn].numpy()
        buf[:lay.total] = 0
        buf[lay.row_req:lay.row_req + Tc] = -1
        for g in range(len(widths)):
            buf[lay.slots[g]:lay.slots[g] + Tc] = -1
            buf[lay.tables[g]:lay.tables[g] + Rc * widths[g]] = -1
        if T == R and _SINGLE_TOKEN_PATH and all(len(e.tokens) == 1 for e in entries):
            # a decoding step: one row a request, so whole columns are written at once
            starts = np.fromiter((e.cache.length for e in entries), dtype=np.int32, count=R)
            rows = np.arange(R, dtype=np.int32)
            state_slots = [e.cache.state_slot for e in entries]
            buf[lay.ids:lay.ids + R] = np.fromiter((e.tokens[0] for e in entries), dtype=np.int32, count=R)
            buf[lay.pos:lay.pos + R] = starts
            buf[lay.row_req:lay.row_req + R] = rows
            buf[lay.q_start:lay.q_start + R] = rows
            buf[lay.kv_len:lay.kv_len + R] = starts + 1
            buf[lay.state_slot:lay.state_slot + R] = state_slots
            wanted = [r for r, e in enumerate(entries) for _ in e.want]
            buf[lay.want:lay.want + len(wanted)] = wanted
            for g in range(len(widths)):
                at, width, slots = lay.tables[g], widths[g], lay.slots[g]
                for r, e in enumerate(entries):
                    table = e.cache.tables[g]
                    buf[at + r * width:at + r * width + len(table)] = table
                    position = e.cache.length
                    buf[slots + r] = table[position // page] * page + position % page
            buf[lay.q_start + R:lay.q_start + Rc + 1] = R
            counts = self._annotate(buf, lay, rows, np.ones(R, dtype=np.int32), starts, padded)
            return PackedStep(lay, turn, widths, Tc, Rc, Wc, W, [1] * R, (starts + 1).tolist(), state_slots,
                              counts)
        q_lens, kv_lens, state_slots = [], [], []
        row = 0
        want_at = 0
        for r, e in enumerate(entries):
            n = len(e.tokens)
            start = e.cache.length
            buf[lay.ids + row:lay.ids + row + n] = np.asarray(e.tokens, dtype=np.int32)
            positions = np.arange(start, start + n, dtype=np.int32)
            buf[lay.pos + row:lay.pos + row + n] = positions
            buf[lay.row_req + row:lay.row_req + row + n] = r
            buf[lay.q_start + r] = row
            buf[lay.kv_len + r] = start + n
            buf[lay.state_slot + r] = e.cache.state_slot
            for w in e.want:
                buf[lay.want + want_at] = row + int(w)
                want_at += 1
            for g in range(len(widths)):
                table = np.asarray(e.cache.tables[g], dtype=np.int32)
                buf[lay.tables[g] + r * widths[g]:lay.tables[g] + r * widths[g] + len(table)] = table
                buf[lay.slots[g] + row:lay.slots[g] + row + n] = \
                    table[positions // page] * page + positions % page
            q_lens.append(n)
            kv_lens.append(start + n)
            state_slots.append(e.cache.state_slot)
            row += n
        buf[lay.q_start + R:lay.q_start + Rc + 1] = row
        q_counts = np.asarray(q_lens, dtype=np.int32)
        first_rows = np.concatenate(([0], np.cumsum(q_counts)[:-1])).astype(np.int32)
        starts = np.asarray(kv_lens, dtype=np.int32) - q_counts
        counts = self._annotate(buf, lay, first_rows, q_counts, starts, padded)
        return PackedStep(lay, turn, widths, Tc, Rc, Wc, W, q_lens, kv_lens, state_slots, counts)

    def _annotate(self, buf, lay: BatchLayout, first_rows, counts, starts, padded: bool) -> List[int]:
        """Let every annotation of the model's parts write its words (the buffer is zeroed)."""
        return [int(note.fill(buf[at:at + words], first_rows, counts, starts, padded))
                for note, at, words in zip(self.annotations, lay.notes, lay.note_words)]

    def set_ids(self, packed: "PackedStep", ids: Sequence[int]) -> None:
        """Put the token ids of a packed step of single tokens in place (row = entry)."""
        lay = packed.layout
        self._hosts[packed.turn].numpy()[lay.ids:lay.ids + len(ids)] = np.asarray(ids, dtype=np.int32)

    def copy_ids(self, packed: "PackedStep", ids: torch.Tensor) -> None:
        """Put token ids that are still on the device (int32, row = entry) in the place of a
        packed step of single tokens, after `copy` and before the step runs."""
        lay = packed.layout
        self._dev[lay.ids:lay.ids + ids.numel()].copy_(ids, non_blocking=True)

    def copy(self, packed: "PackedStep") -> int:
        """Only the copy to the device (a replayed graph has the views baked in); returns the
        number of wanted rows."""
        lay = packed.layout
        dev, host = self._dev, self._hosts[packed.turn]
        dev[:lay.total].copy_(host[:lay.total], non_blocking=True)
        self.last_bytes = lay.total * 4
        if dev.is_cuda:
            self._copied[packed.turn] = torch.cuda.Event()
            self._copied[packed.turn].record()
        return packed.n_want

    def upload(self, packed: "PackedStep"):
        """The device's half: one copy, and the views the parts receive."""
        lay, widths = packed.layout, packed.widths
        Tc, Rc, Wc = packed.tokens, packed.requests, packed.wanted
        dev = self._dev
        page = self.plan.page_size
        self.copy(packed)

        def view(offset, n):
            return dev[offset:offset + n]

        groups = [GroupView(page, view(lay.slots[g], Tc),
                            view(lay.tables[g], Rc * widths[g]).view(Rc, widths[g]))
                  for g in range(len(widths))]
        ctx = StepContext(
            n_tokens=Tc, n_requests=Rc, ids=view(lay.ids, Tc), pos=view(lay.pos, Tc),
            row_req=view(lay.row_req, Tc), q_start=view(lay.q_start, Rc + 1),
            kv_len=view(lay.kv_len, Rc), state_slot=view(lay.state_slot, Rc), groups=groups,
            q_lens=packed.q_lens, kv_lens=packed.kv_lens, state_slots=packed.state_slots,
            views={note.key: (note.view(view(at, words)), count)
                   for note, at, words, count in zip(self.annotations, lay.notes, lay.note_words,
                                                     packed.note_counts)})
        return ctx, view(lay.want, Wc), packed.n_want

"""Request options, the per-request sampling cursor and the result record, in
the reference's names and meanings (qwen-infer/src/generate.rs:16-101, 167-338,
409-501; stream.rs:11-78)."""
from __future__ import annotations

import codecs
import enum
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..sampling.rng import uniform
from ..sampling.sampler import validate_sampling


class StopReason(enum.Enum):
    MAX_TOKENS = "max_tokens"      # max_tokens ids were sampled, none of them EOS
    EOS = "eos"                    # the sampled id is in `eos`; it is not kept
    STOP_STRING = "stop_string"    # a stop string occurred in the decoded text
    CANCELLED = "cancelled"        # the chunk callback asked to stop
    FAILED = "failed"              # the request could not be run (see `error`)


class Control(enum.Enum):
    CONTINUE = 0
    STOP = 1


@dataclass
class GenerateParams:
    max_tokens: int = 20
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0
    eos: Sequence[int] = ()
    stop: Sequence[str] = ()

    @classmethod
    def greedy(cls, max_tokens: int) -> "GenerateParams":
        return cls(max_tokens=max_tokens)

    def validate(self) -> None:
        validate_sampling(self.temperature, self.top_p)
        if self.max_tokens < 0:
            raise ValueError("max_tokens is negative")
        if any(s == "" for s in self.stop):
            raise ValueError("stop strings must be non-empty")


@dataclass
class Generated:
    tokens: List[int]
    text: str
    chunks: List[str]
    reason: StopReason
    completion_tokens: int
    prefill: float = 0.0       # seconds until the prompt was run
    decode: float = 0.0        # seconds from then to the end
    error: Optional[str] = None


class StreamDecoder:
    """Bytes of tokens to text: an unfinished UTF-8 tail waits for the next
    token; a complete illegal sequence becomes U+FFFD; `finish` turns a tail
    that never completed into U+FFFD."""

    def __init__(self):
        self._decoder = codecs.getincrementaldecoder("utf-8")(errors="replace")

    def push(self, data: bytes) -> str:
        return self._decoder.decode(data, final=False)

    def finish(self) -> str:
        return self._decoder.decode(b"", final=True)


class StopHold:
    """Decoded text and how much of it was handed out.  A suffix that is a
    proper prefix of a stop string is held back until the next piece decides."""

    def __init__(self):
        self.full = ""
        self.emitted = 0

    def push(self, piece: str, stops: Sequence[str]):
        """Returns (stopped, text to emit)."""
        self.full += piece
        found = [self.full.find(s) for s in stops]
        found = [f for f in found if f >= 0]
        if found:
            at = min(found)
            emit = self.full[self.emitted:at] if at > self.emitted else ""
            self.emitted = at
            return True, emit
        hold = 0
        for s in stops:
            for n in range(1, min(len(self.full), len(s) - 1) + 1):
                if self.full.endswith(s[:n]):
                    hold = max(hold, n)
        safe = len(self.full) - hold
        if safe < self.emitted:
            return False, ""
        emit = self.full[self.emitted:safe]
        self.emitted = safe
        return False, emit

    def finish(self) -> str:
        emit = self.full[self.emitted:]
        self.emitted = len(self.full)
        return emit


class SampleCursor:
    """One request's sampling state.  The scheduler draws ids on the device
    (with this cursor's temperature, top_p and next uniform) and hands each to
    `accept`, which answers whether to run the id forward or to finish."""

    def __init__(self, params: GenerateParams,
                 token_bytes: Optional[Callable[[int], bytes]] = None,
                 on_chunk: Optional[Callable[[str], Control]] = None):
        params.validate()
        if params.stop and token_bytes is None:
            raise ValueError("stop strings need a tokenizer (token ids -> bytes)")
        self.params = params
        self.token_bytes = token_bytes
        self.on_chunk = on_chunk
        self.decoder = StreamDecoder()
        self.held = StopHold()
        self.tokens: List[int] = []
        self.chunks: List[str] = []
        self.text = ""
        self.produced = 0
        self.drawn = 0
        self.done: Optional[Generated] = None

    def wants_sample(self) -> bool:
        """False when max_tokens is already met (generate.rs:238-242)."""
        if self.done is None and self.produced >= self.params.max_tokens:
            self._finish(StopReason.MAX_TOKENS)
        return self.done is None

    def next_uniform(self) -> float:
        """The draw for the next id; the greedy choice uses none (sample.rs:43-56)."""
        if self.params.temperature == 0:
            return 0.0
        return uniform(self.params.seed, self.drawn)

    def _observe(self, piece: str) -> Control:
        if piece:
            self.chunks.append(piece)
            self.text += piece
        if self.on_chunk is None:
            return Control.CONTINUE
        return self.on_chunk(piece) or Control.CONTINUE

    def _snapshot(self, reason: StopReason) -> Generated:
        self.done = Generated(list(self.tokens), self.text, list(self.chunks), reason,
                              self.produced)
        return self.done

    def _finish(self, reason: StopReason) -> Generated:
        # generate.rs:303-338: MaxTokens and Eos flush the decoder and the hold
        flushed = self.decoder.finish() if self.token_bytes else ""
        if flushed:
            stopped, emit = self.held.push(flushed, self.params.stop)
            if stopped:
                control = self._observe(emit)
                reason = StopReason.CANCELLED if control == Control.STOP else StopReason.STOP_STRING
            else:
                first = self._observe(emit)
                second = self._observe(self.held.finish())
                if Control.STOP in (first, second):
                    reason = StopReason.CANCELLED
        else:
            if self._observe(self.held.finish()) == Control.STOP:
                reason = StopReason.CANCELLED
        return self._snapshot(reason)

    def accept(self, token: int) -> bool:
        """Take the id just drawn.  True: run it forward; False: finished
        (`self.done` holds the result).  generate.rs:243-283."""
        self.drawn += 1
        if token in self.params.eos:
            self.produced += 1
            self._finish(StopReason.EOS)
            return False
        piece = self.decoder.push(self.token_bytes(token)) if self.token_bytes else ""
        stopped, emit = self.held.push(piece, self.params.stop)
        self.tokens.append(token)
        self.produced += 1
        control = self._observe(emit)
        if stopped:
            self._snapshot(StopReason.CANCELLED if control == Control.STOP else StopReason.STOP_STRING)
            return False
        if control == Control.STOP:
            self._snapshot(StopReason.CANCELLED)
            return False
        if self.produced >= self.params.max_tokens:
            self._finish(StopReason.MAX_TOKENS)
            return False
        return True

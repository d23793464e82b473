"""What every part is built from: the registries, the runtime (device and
precision), the description of one step's batch that parts receive, the cache
needs a mixer declares and the residual stream with its pending add.

A part never knows which model it is in.  It is built from a `PartSpec` (sizes
and constants as parameters, a prefix for its tensors), declares its tensors
with `tensors(spec)` and works on the rows it is handed.

Interfaces (duck-typed; the classes below marked "interface" document them):

  mixer         tensors(spec); __init__(spec, store, runtime); cache_need();
                forward(h [T,H], ctx: StepContext, cache: CacheBinding) -> delta
                optional: batch_annotations() -> [BatchAnnotation] (integer data about the
                batch that its kernels want packed with the step), shape_key(q_lens) -> hashable
                (what, beyond the step's sizes, decides which kernels it launches: part of a
                captured graph's key), advance_decode(ctx, cache) (move per-request state on
                after a device-side decoding step), graph_safe = True (launches depend on
                device-side metadata only)
  feed_forward  tensors(spec); __init__(spec, store, runtime); forward(h [T,H]) -> delta
                (delta is [T,H] in the compute dtype, or float32 partial sums [S,T,H]
                that the residual stream adds up in index order)
  norm          tensors(spec); __init__(spec, store, runtime);
                forward(x f32 [T,H], delta=None, rows=None) -> h (compute dtype)
  position      tensors(spec); __init__(spec, store, runtime); tables used by the mixer
  block         PARTS = {name: category}; __init__(**parts by those names), kept as attributes
                of those names (`mixer` is the part whose cache need the cache manager
                serves); forward(stream, ctx, cache)
  embedding     forward(ids) -> x f32 [T,H];   head  forward(stream, rows) -> logits f32
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..config.spec import ConfigError, PartSpec
from ..kernels import ops

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_REGISTRY: Dict[str, Dict[str, Any]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls: Any) -> None:
    """Make `cls` buildable from a PartSpec of this `kind`."""
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")
    _REGISTRY[category][kind] = cls


def part_class(category: str, kind: str) -> Any:
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY[category])) or "none"
        raise ConfigError(f"no {category} of kind {kind!r} is registered (registered: {known})") from None


def registered(category: str) -> List[str]:
    return sorted(_REGISTRY[category])


# --------------------------------------------------------------------------- #
@dataclass
class Runtime:
    """Where and in which precision a model runs.  `dtype` is the type of the
    matrix-product operands and of the cache: bfloat16 for serving, float32
    for the true 32-bit path.  The residual stream, norm gains, biases and
    logits are float32 in both."""

    device: torch.device
    dtype: torch.dtype

    def __post_init__(self):
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype is float32 or bfloat16, found {self.dtype}")

    def matrix(self, stored: torch.Tensor) -> torch.Tensor:
        """A matrix-product operand in the compute dtype, on the device."""
        return stored.to(device=self.device, dtype=self.dtype).contiguous()

    def vector(self, stored: torch.Tensor) -> torch.Tensor:
        """A gain or bias: widened to float32 (exact for bfloat16)."""
        return stored.to(device=self.device, dtype=torch.float32).contiguous()

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class KVNeed:
    """Keys and values per token: `kv_heads` x `head_dim` each.  With a
    `window`, only the last window + 1 positions are ever read, and pages
    wholly before them are given back."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size per request (float32), zeroed when a request starts."""

    shape: Tuple[int, ...]


@dataclass(frozen=True)
class CacheNeed:
    kv: Optional[KVNeed] = None
    state: Optional[StateNeed] = None


@dataclass
class GroupView:
    """The batch as one cache group sees it: where each row's keys go and the
    block table of each request (logical block -> page, -1 where none)."""

    page_size: int
    slots: torch.Tensor          # [T] int32: page * page_size + offset
    block_table: torch.Tensor    # [R, max_blocks] int32


@dataclass
class StepContext:
    """One step's batch, as parts see it: T rows of R requests.  Row t belongs
    to request `row_req[t]` and sits at absolute position `pos[t]`; a request's
    rows are contiguous and in order (`q_start[r]` .. `q_start[r+1]`)."""

    n_tokens: int
    n_requests: int
    ids: torch.Tensor            # [T] int32
    pos: torch.Tensor            # [T] int32
    row_req: torch.Tensor        # [T] int32
    q_start: torch.Tensor        # [R + 1] int32
    kv_len: torch.Tensor         # [R] int32, tokens held after this step
    state_slot: torch.Tensor     # [R] int32
    groups: List[GroupView]
    # what the model's parts asked to have packed with the batch (`BatchAnnotation`), by key:
    # (the annotation's device view, the count its `fill` returned)
    views: Dict[str, Tuple[Any, int]] = field(default_factory=dict)
    # the block that runs after the one running now (None after the last): a part that asks for
    # memory ahead of its use may look at what that block starts with
    next_block: Any = None
    # host copies, for choosing kernels and for mixers that loop over requests
    q_lens: List[int] = field(default_factory=list)
    kv_lens: List[int] = field(default_factory=list)
    state_slots: List[int] = field(default_factory=list)

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens) if self.q_lens else 0

    @property
    def max_kv_len(self) -> int:
        return max(self.kv_lens) if self.kv_lens else 0


class BatchAnnotation:
    """Interface.  Integer data about a step's batch that a part's kernels want beside the
    rows, positions and tables every part gets: a cut of the rows into tiles, a schedule, a
    sorted order.  A part lists its annotations in `batch_annotations()`; the engine packs each
    (once per `key`, however many layers ask) into the step's one metadata buffer, at an
    offset that depends on the step's capacities only, so a captured graph finds it again; the
    part reads `ctx.views[key]`.  The batch builder knows none of them.

      key                         a string; equal keys are one annotation
      capacity(T, R) -> int       int32 words for a step of up to T rows of R requests
      fill(out, first_rows, counts, starts, padded) -> int
                                  write the step's data into `out` (a zeroed numpy int32 array of
                                  `capacity` words) from the requests' spans: request r brings
                                  rows first_rows[r] .. + counts[r], the first at position
                                  starts[r] (numpy arrays).  `padded`: the step will be replayed
                                  from a graph, so the count returned must be the most the
                                  capacities allow.  The count travels with the view.
      view(words) -> Any          the device-side int32 words (a tensor of `capacity`) as the
                                  part wants to see them
    """

    key = ""

    def capacity(self, n_tokens: int, n_requests: int) -> int:
        raise NotImplementedError

    def fill(self, out, first_rows, counts, starts, padded: bool) -> int:
        raise NotImplementedError

    def view(self, words):
        return words


@dataclass
class CacheBinding:
    """What one call of a mixer may touch in the cache.  `writes` is False when
    the call reads the cache that an earlier call wrote."""

    group: int = -1                           # index into StepContext.groups, -1: no keys
    k_pool: Optional[torch.Tensor] = None     # [pages * page_size, kv_heads, head_dim]
    v_pool: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None      # [state slots, *shape] float32
    writes: bool = True


# --------------------------------------------------------------------------- #
class ResidualStream:
    """The residual sum, kept in float32.  A part's output is not added at once:
    it stays pending until the next norm, which adds it while it reads the row
    (one pass over memory instead of two)."""

    def __init__(self, x: torch.Tensor):
        if x.dtype != torch.float32:
            raise ValueError("the residual stream is float32")
        self.x = x
        self.pending: Optional[torch.Tensor] = None

    def add(self, delta: torch.Tensor) -> None:
        self.flush()
        self.pending = delta

    def flush(self) -> torch.Tensor:
        if self.pending is not None:
            ops.residual_add(self.x, self.pending)
            self.pending = None
        return self.x

    def normed(self, norm) -> torch.Tensor:
        delta, self.pending = self.pending, None
        return norm.forward(self.x, delta=delta)


def build_part(category: str, spec: PartSpec, store, runtime: Runtime):
    return part_class(category, spec.kind)(spec, store, runtime)

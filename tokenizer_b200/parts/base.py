"""What every part is built from: the registries, the runtime (device and
precision), the description of one step's batch that parts receive, the cache
needs a mixer declares and the residual stream with its pending add.

A part never knows which model it is in.  It is built from a `PartSpec` (sizes
and constants as parameters, a prefix for its tensors), declares its tensors
with `tensors(spec)` and works on the rows it is handed.

Interfaces (duck-typed; the classes below marked "interface" document them):

  mixer         tensors(spec); __init__(spec, store, runtime); cache_need();
                forward(h [T,H], ctx: StepContext, cache: CacheBinding) -> delta
  feed_forward  tensors(spec); __init__(spec, store, runtime); forward(h [T,H]) -> delta
                (delta is [T,H] in the compute dtype, or float32 partial sums [S,T,H]
                that the residual stream adds up in index order)
  norm          tensors(spec); __init__(spec, store, runtime);
                forward(x f32 [T,H], delta=None, rows=None) -> h (compute dtype)
  position      tensors(spec); __init__(spec, store, runtime); tables used by the mixer
  block         __init__(layer_spec, parts, runtime); forward(stream, ctx, cache)
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
    # the rows cut into tiles of up to 64 consecutive rows of one request:
    # int32 [n_q_tiles, 2] = (first row, rows); None when the builder made none
    q_tiles: Optional[torch.Tensor] = None
    n_q_tiles: int = 0
    # the same cut into tiles of up to 128 rows (the tcgen05 attention kernel's tile)
    q_wide_tiles: Optional[torch.Tensor] = None
    n_q_wide_tiles: int = 0
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

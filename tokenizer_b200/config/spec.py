"""Architecture-neutral description of a decoder, produced by a typed config.

A typed configuration (one class per architecture, see `qwen2.py`) reads the
architecture's own `config.json` keys and turns them into a `ModelSpec`: plain
data that names, layer by layer, which mixer, feed-forward, norm and position
encoding to build and with which sizes and constants.  Everything below the
configuration (parts, cache manager, step function, scheduler) sees only this
data, never the architecture.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a model this framework can run."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the `kind` names a registered part class, `params`
    are the sizes and constants its constructor takes, `prefix` is where its
    tensors live in the weight file ("model.layers.3.self_attn")."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""

    def with_prefix(self, prefix: str) -> "PartSpec":
        return PartSpec(self.kind, dict(self.params), prefix)


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: how its parts are arranged (`block`, e.g. pre-norm
    residual), the token mixer, the feed-forward and the two norms."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.  `layer` indexes `ModelSpec.layers`.
    `cache` names the cache slot the mixer uses at this call: by default a slot
    of its own (the index of the call in the order); the index of an earlier
    call makes the mixer read that call's cache instead of writing one."""

    layer: int
    cache: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec

    def validate(self) -> None:
        if not self.layers or not self.order:
            raise ConfigError("a model needs at least one layer and one call in its order")
        for at, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ConfigError(f"order[{at}] names layer {call.layer}, there are {len(self.layers)}")
            if call.cache is not None and not 0 <= call.cache < at:
                raise ConfigError(
                    f"order[{at}] reads the cache of call {call.cache}, which does not run before it"
                )
            if call.cache is not None and self.order[call.cache].cache is not None:
                raise ConfigError(f"order[{at}] reads call {call.cache}, which owns no cache itself")


def require_keys(raw: Dict[str, Any], keys: List[str], what: str) -> None:
    missing = [k for k in keys if k not in raw]
    if missing:
        raise ConfigError(f"{what}: config.json lacks {', '.join(missing)}")


def as_int(raw: Dict[str, Any], key: str, minimum: int = 0) -> int:
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json {key} must be an integer, found {value!r}")
    if value < minimum:
        raise ConfigError(f"config.json {key} must be at least {minimum}, found {value}")
    return value


def as_float(raw: Dict[str, Any], key: str) -> float:
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json {key} must be a number, found {value!r}")
    return float(value)


def as_bool(raw: Dict[str, Any], key: str) -> bool:
    value = raw[key]
    if not isinstance(value, bool):
        raise ConfigError(f"config.json {key} must be true or false, found {value!r}")
    return value

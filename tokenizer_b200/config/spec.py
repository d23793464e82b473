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


class LayerSpec:
    """One decoder layer: `block` names a registered arrangement (e.g. pre-norm residual) and
    `parts` are the parts it arranges, by name.  The arrangement's class says which names it
    wants and of which category each is (its `PARTS`), so another arrangement (a third norm,
    two mixers side by side, no feed-forward) is a new registered block and nothing else.
    The four names of the pre-norm residual block can be given positionally; every name is
    also an attribute (`layer.mixer`)."""

    def __init__(self, block: str, mixer: Optional[PartSpec] = None,
                 feed_forward: Optional[PartSpec] = None, mixer_norm: Optional[PartSpec] = None,
                 feed_forward_norm: Optional[PartSpec] = None, **more: PartSpec):
        parts: Dict[str, PartSpec] = {}
        for name, spec in (("mixer", mixer), ("feed_forward", feed_forward),
                           ("mixer_norm", mixer_norm), ("feed_forward_norm", feed_forward_norm)):
            if spec is not None:
                parts[name] = spec
        parts.update(more)
        for name, spec in parts.items():
            if not isinstance(spec, PartSpec):
                raise ConfigError(f"layer part {name!r} must be a PartSpec, found {type(spec).__name__}")
        self.block = block
        self.parts = parts

    def __getattr__(self, name: str) -> PartSpec:
        parts = self.__dict__.get("parts", {})
        if name in parts:
            return parts[name]
        raise AttributeError(f"this layer has no part named {name!r} (it has {', '.join(parts) or 'none'})")

    def __repr__(self) -> str:
        return f"LayerSpec({self.block!r}, {self.parts!r})"


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

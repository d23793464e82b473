"""The one registry from an architecture's name to its typed configuration.

`config.json["architectures"][0]` chooses the entry everywhere: loading a
folder, random weights, replay, generation.  An entry is the configuration
class; the class reads its own keys (`from_dict`) and describes the model as a
`ModelSpec` (`model_spec`), from which the generic decoder is assembled.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Type

from .spec import ConfigError

_ARCHITECTURES: Dict[str, Type] = {}


def register_architecture(name: str, config_class: Type) -> None:
    """Add an architecture.  `config_class` needs `from_dict(dict)`,
    `to_dict()` and `model_spec()`."""
    for method in ("from_dict", "to_dict", "model_spec"):
        if not hasattr(config_class, method):
            raise TypeError(f"{config_class.__name__} lacks {method}()")
    _ARCHITECTURES[name] = config_class


def registered_architectures():
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> Type:
    if name not in _ARCHITECTURES:
        known = ", ".join(registered_architectures()) or "none"
        raise ConfigError(f"architecture {name!r} is not registered (registered: {known})")
    return _ARCHITECTURES[name]


def config_from_dict(raw: Dict[str, Any]):
    names = raw.get("architectures")
    if not isinstance(names, list) or not names or not isinstance(names[0], str):
        raise ConfigError('config.json needs "architectures": ["<name>"]')
    return config_class_for(names[0]).from_dict(raw)


def load_config(folder: str):
    path = os.path.join(folder, "config.json")
    try:
        with open(path) as fh:
            raw = json.load(fh)
    except FileNotFoundError:
        raise ConfigError(f"{path} does not exist") from None
    except json.JSONDecodeError as err:
        raise ConfigError(f"{path} is not JSON: {err}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return config_from_dict(raw)

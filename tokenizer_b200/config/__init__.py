from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec
from .registry import (config_class_for, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .qwen2 import Qwen2Config

__all__ = [
    "ConfigError", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec", "Qwen2Config",
    "config_class_for", "config_from_dict", "load_config", "register_architecture",
    "registered_architectures",
]

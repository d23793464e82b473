"""tokenizer_b200: a small, whole inference engine for one GPU (NVIDIA B200,
sm_100a): from a model folder (config.json, model.safetensors) to the next
token.  See `generate` for the entry point."""
from .config import ConfigError, Qwen2Config, load_config, register_architecture
from .weights import WeightError, write_random_model

__all__ = ["ConfigError", "Qwen2Config", "WeightError", "load_config", "register_architecture",
           "write_random_model"]
__version__ = "0.1.0"

"""tokenizer_b200: a small, whole inference engine for one GPU (NVIDIA B200,
sm_100a): from a model folder (config.json, model.safetensors) to the next
token.  See `generate` for the entry point."""
from . import config
from .config import ConfigError, Qwen2Config, load_config, register_architecture
from .weights import WeightError, write_random_model

from .api import (Control, Engine, Generated, GenerateParams, StopReason, engine_for, generate,
                  generate_batch, generate_with, greedy_tokens, load_eos_token_ids, load_model, random_model)
from .engine.scheduler import Scheduler

__all__ = ["Control", "Engine", "Generated", "GenerateParams", "StopReason", "engine_for",
           "generate", "generate_batch", "generate_with", "greedy_tokens", "load_eos_token_ids",
           "load_model", "random_model", "Scheduler", "ConfigError", "Qwen2Config", "WeightError", "load_config", "register_architecture",
           "write_random_model"]
__version__ = "0.1.0"

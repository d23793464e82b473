from .batch import StepEntry
from .step import Engine, load_model, parse_dtype

__all__ = ["Engine", "StepEntry", "load_model", "parse_dtype"]

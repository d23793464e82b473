from .safetensors_io import WeightError, read_safetensors, write_safetensors
from .store import TensorSpec, WeightStore
from .random_init import SeededTensors, random_tensors, write_random_model

__all__ = ["SeededTensors", "TensorSpec", "WeightError", "WeightStore", "random_tensors", "read_safetensors",
           "write_random_model", "write_safetensors"]

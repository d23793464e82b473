from .rng import uniform
from .sampler import Sampler, validate_sampling

__all__ = ["Sampler", "uniform", "validate_sampling"]

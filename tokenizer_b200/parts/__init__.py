from .base import (BatchAnnotation, CacheBinding, CacheNeed, GroupView, KVNeed, ResidualStream, Runtime, StateNeed,
                   StepContext, build_part, part_class, register_part, registered)
from . import attention, block, embedding, feed_forward, norm, position  # register the parts
from .linear import Linear
from .model import DecoderModel, declared_tensors

__all__ = ["BatchAnnotation", "CacheBinding", "CacheNeed", "DecoderModel", "GroupView", "KVNeed", "Linear",
           "ResidualStream", "Runtime", "StateNeed", "StepContext", "build_part",
           "declared_tensors", "part_class", "register_part", "registered"]

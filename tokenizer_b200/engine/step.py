"""The engine and its one step function.

`Engine.step(entries)` runs a batch of (request, its next tokens): portions of
prompts beside single decoded tokens, cut anywhere.  It runs only the tokens it
is given, as one batch, against the cache that earlier steps left, writes their
keys and values into the pages reserved for them, and returns the float32
logits at the wanted places.  Pages are reserved by the caller (the scheduler
or the replay program) through `engine.cache`; the step itself allocates none,
as the reference's paged forwards do not (qwen-infer/src/model.rs:1015-1053).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.device import DeviceCache
from ..config.registry import load_config
from ..kernels.ops import KernelError
from ..parts.base import Runtime
from ..parts.model import DecoderModel
from ..weights.store import WeightStore
from ..sampling.sampler import Sampler
from .batch import BatchBuilder, StepEntry

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _DTYPES[str(name)]
    except KeyError:
        raise ValueError(f"dtype is bfloat16 or float32, found {name!r}") from None


def load_model(folder: str, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """Build the model that the folder's config.json names, with the folder's
    weights, on `device`.  There is no CPU path."""
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise KernelError(
            "tokenizer_b200 runs on a CUDA GPU (sm_100a) only; no GPU is visible to this process")
    config = load_config(folder)
    store = WeightStore.from_folder(folder)
    with torch.cuda.device(device):
        model = DecoderModel(config.model_spec(), store, Runtime(device, parse_dtype(dtype)))
    model.config = config
    return model


class Engine:
    def __init__(self, model: DecoderModel, num_pages: int, page_size: int = 16,
                 max_requests: int = 64, share_prefixes: bool = False):
        self.model = model
        self.runtime = model.runtime
        self.cache = DeviceCache(model.cache_needs(), num_pages, page_size, max_requests,
                                 model.runtime, share_prefixes)
        self.bindings = self.cache.bindings(model.order)
        self.builder = BatchBuilder(self.cache, model.vocab_size, model.max_positions,
                                    model.runtime.device)
        self.sampler = Sampler(model.runtime.device)
        self.max_positions = model.max_positions
        self.steps_run = 0

    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0", **kw) -> "Engine":
        return cls(load_model(folder, dtype, device), **kw)

    def step(self, entries: List[StepEntry]) -> torch.Tensor:
        """Run one batch; returns logits [wanted, vocab] float32 on the device,
        in the order of the entries and of their `want`."""
        if not entries:
            return torch.empty((0, self.model.vocab_size), dtype=torch.float32,
                               device=self.runtime.device)
        self.builder.validate(entries)
        with torch.cuda.device(self.runtime.device):
            ctx, want_rows, n_want = self.builder.build(entries)
            logits = self.model.forward(ctx, self.bindings, want_rows[:n_want])
        for e in entries:
            self.cache.commit(e.cache, len(e.tokens))
        self.steps_run += 1
        return logits

    def sample(self, logits: torch.Tensor, temperature, top_p, uniform) -> List[int]:
        """Draw one id per row of `logits` on the device."""
        with torch.cuda.device(self.runtime.device):
            return self.sampler.sample(logits, temperature, top_p, uniform)

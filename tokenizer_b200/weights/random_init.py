"""Random-weights mode: write a model folder (config.json, model.safetensors)
from a configuration and a seed.  Linear weights, embeddings and biases are
N(0, 0.02), norm gains 1 + N(0, 0.02), all stored in bfloat16 as released
checkpoints are.  Tensors are drawn in sorted-name order from one generator, so
a folder is a function of (configuration, seed) alone."""
from __future__ import annotations

import json
import os
import re
from typing import Dict, Optional

import torch

from .safetensors_io import write_safetensors


def random_tensors(specs, seed: int, scale: Optional[Dict[str, float]] = None,
                   dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """`scale` maps a regular expression over tensor names to a factor applied
    to the drawn values (tests sharpen attention by scaling q and k)."""
    generator = torch.Generator(device="cpu")
    generator.manual_seed(int(seed))
    tensors = {}
    for spec in sorted(specs, key=lambda s: s.name):
        if spec.init == "zeros":
            value = torch.zeros(spec.shape, dtype=torch.float32)
        else:
            value = torch.randn(spec.shape, generator=generator, dtype=torch.float32) * spec.std
            if spec.init == "one_plus_normal":
                value = value + 1.0
            elif spec.init != "normal":
                raise ValueError(f"tensor {spec.name}: unknown init {spec.init!r}")
        for pattern, factor in (scale or {}).items():
            if re.search(pattern, spec.name):
                value = value * factor
        tensors[spec.name] = value.to(dtype)
    return tensors


class SeededTensors:
    """A model's random weights without a file: a mapping from tensor name to a tensor drawn
    when it is asked for, on `device`, from a generator seeded by (seed, name), so that a
    tensor is a function of the configuration, the seed and its own name alone.  For models
    whose weights would be many gigabytes on disk (a benchmark at 7B sizes); `WeightStore`
    takes it in place of a dict.  The values differ from `write_random_model`'s (one
    generator on the CPU, in sorted-name order): the two modes do not mix."""

    def __init__(self, specs, seed: int, device="cpu", dtype: torch.dtype = torch.bfloat16):
        self.specs = {spec.name: spec for spec in specs}
        self.seed, self.device, self.dtype = int(seed), torch.device(device), dtype

    def __contains__(self, name) -> bool:
        return name in self.specs

    def __iter__(self):
        return iter(self.specs)

    def __len__(self) -> int:
        return len(self.specs)

    def shape_of(self, name: str):
        return tuple(self.specs[name].shape)

    def __getitem__(self, name: str) -> torch.Tensor:
        import zlib
        spec = self.specs[name]
        if spec.init == "zeros":
            return torch.zeros(spec.shape, dtype=self.dtype, device=self.device)
        generator = torch.Generator(device=self.device)
        generator.manual_seed((self.seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF)
        value = torch.randn(spec.shape, generator=generator, dtype=torch.float32, device=self.device) * spec.std
        if spec.init == "one_plus_normal":
            value = value + 1.0
        elif spec.init != "normal":
            raise ValueError(f"tensor {spec.name}: unknown init {spec.init!r}")
        return value.to(self.dtype)


def write_random_model(folder: str, config, seed: int,
                       scale: Optional[Dict[str, float]] = None,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Create `folder` with config.json and model.safetensors for `config`
    (a registered typed configuration)."""
    from ..parts.model import declared_tensors  # parts declare what they need

    os.makedirs(folder, exist_ok=True)
    specs = declared_tensors(config.model_spec())
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(specs, seed, scale, dtype))
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(config.to_dict(), fh, indent=1)
    return folder

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

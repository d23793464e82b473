"""Weights by tensor name.

Parts declare the tensors they need (`TensorSpec`: name, shape, how random
mode draws it).  `WeightStore.check` compares the whole declaration with the
file once and raises ONE error that lists every missing tensor, every
unexpected tensor and every wrong shape.  Stored precision is kept: bfloat16
stays bfloat16 (float16 is brought to bfloat16), integer tables become int32,
and a tensor stored in 32-bit stays 32-bit.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

from .safetensors_io import WeightError, read_safetensors


@dataclass(frozen=True)
class TensorSpec:
    """`init` tells random-weights mode what to draw: "normal" (mean 0),
    "one_plus_normal" (norm gains), "zeros"; `std` is its scale."""

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    std: float = 0.02


def _keep_precision(tensor: torch.Tensor) -> torch.Tensor:
    if tensor.dtype in (torch.bfloat16, torch.float32, torch.int32):
        return tensor
    if tensor.dtype == torch.float16:
        return tensor.to(torch.bfloat16)
    if tensor.dtype == torch.float64:
        return tensor.to(torch.float32)
    if tensor.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool):
        return tensor.to(torch.int32)
    raise WeightError(f"dtype {tensor.dtype} has no place in a model")


class WeightStore:
    def __init__(self, tensors: Dict[str, torch.Tensor], source: str = "<memory>"):
        self.tensors = tensors
        self.source = source

    @classmethod
    def from_folder(cls, folder: str) -> "WeightStore":
        """`model.safetensors`, or the files that `model.safetensors.index.json` names (its
        "weight_map": tensor name -> file).  A tensor that the index sends to a file which does
        not hold it counts as missing; one that two files hold is an error here."""
        path = os.path.join(folder, "model.safetensors")
        index = os.path.join(folder, "model.safetensors.index.json")
        if os.path.exists(path) or not os.path.exists(index):
            return cls(read_safetensors(path), path)
        try:
            with open(index) as f:
                weight_map = json.load(f)["weight_map"]
            files = sorted(set(weight_map.values()))
        except (OSError, ValueError, KeyError, TypeError, AttributeError) as err:
            raise WeightError(f"{index}: no usable \"weight_map\" ({err})")
        tensors: Dict[str, torch.Tensor] = {}
        for name in files:
            if not isinstance(name, str) or os.path.basename(name) != name:
                raise WeightError(f"{index}: {name!r} is not a file name inside the folder")
            for key, tensor in read_safetensors(os.path.join(folder, name)).items():
                if key in tensors:
                    raise WeightError(f"{index}: tensor {key} is stored in more than one file")
                tensors[key] = tensor
        return cls(tensors, index)

    def names(self) -> List[str]:
        return sorted(self.tensors)

    def check(self, specs: Iterable[TensorSpec], ignorable: Iterable[str] = ()) -> None:
        """Raise one WeightError naming all that is missing, unexpected or
        mis-shaped.  `ignorable` names tensors a file may carry without use
        (a stored `lm_head.weight` beside a tied head)."""
        wanted = {spec.name: tuple(spec.shape) for spec in specs}
        ignorable = set(ignorable)
        missing = sorted(name for name in wanted if name not in self.tensors)
        unexpected = sorted(
            name for name in self.tensors if name not in wanted and name not in ignorable)
        wrong = sorted(
            (name, self._shape(name), shape)
            for name, shape in wanted.items()
            if name in self.tensors and self._shape(name) != shape)
        if not (missing or unexpected or wrong):
            return
        lines = [f"{self.source} does not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        for name, found, shape in wrong:
            lines.append(f"  wrong shape: {name} is {list(found)}, the model needs {list(shape)}")
        raise WeightError("\n".join(lines))

    def _shape(self, name: str) -> Tuple[int, ...]:
        """A tensor's shape; a source that makes tensors on demand tells it without making one."""
        shape_of = getattr(self.tensors, "shape_of", None)
        return tuple(shape_of(name)) if shape_of is not None else tuple(self.tensors[name].shape)

    def get(self, name: str) -> torch.Tensor:
        """The tensor as stored (see `_keep_precision`), on the CPU."""
        if name not in self.tensors:
            raise WeightError(f"{self.source} has no tensor {name}")
        return _keep_precision(self.tensors[name])

"""Rotary position encoding, half-split form: lane i of a head pairs with lane
i + rotary_dim/2.  inv_freq_i = 1 / theta^(2i / rotary_dim) is computed in
float64 and stored in float32; the angle float32(position) * inv_freq_i and its
cosine and sine are float32 tables of `max_positions` rows
(reference: qwen-infer/src/model.rs:138-172)."""
from __future__ import annotations

import torch

from ..config.spec import ConfigError
from ..kernels import ops
from .base import register_part


class RotaryHalfSplit:
    @staticmethod
    def tensors(spec):
        return []

    def __init__(self, spec, store, runtime):
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        self.max_positions = int(spec.params["max_positions"])
        if self.rotary_dim % 2 or self.rotary_dim <= 0:
            raise ConfigError(f"rotary width {self.rotary_dim} must be even and positive")
        inv_freq = [1.0 / (self.theta ** (i / self.rotary_dim)) for i in range(0, self.rotary_dim, 2)]
        self.inv_freq = torch.tensor(inv_freq, dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.cos, self.sin = ops.rope_table(self.inv_freq, self.max_positions)

    def key(self):
        return (self.theta, self.rotary_dim, self.max_positions)


register_part("position", "rope_half_split", RotaryHalfSplit)

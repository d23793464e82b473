"""Gated feed-forward: down(act(gate(x)) * up(x)), no biases; the gate and up
products are one stacked product (reference: qwen-infer/src/model.rs:226-250,
silu(z) = z * sigmoid(z))."""
from __future__ import annotations

import torch

from ..config.spec import ConfigError
from ..kernels import ops
from ..weights.store import TensorSpec
from .base import register_part
from .linear import Linear


class GatedMLP:
    @staticmethod
    def tensors(spec):
        p, x = spec.params, spec.prefix
        return [
            TensorSpec(x + ".gate_proj.weight", (p["intermediate_size"], p["hidden_size"])),
            TensorSpec(x + ".up_proj.weight", (p["intermediate_size"], p["hidden_size"])),
            TensorSpec(x + ".down_proj.weight", (p["hidden_size"], p["intermediate_size"])),
        ]

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        if p["activation"] != "silu":
            raise ConfigError(f"gated feed-forward knows the silu activation, found {p['activation']}")
        self.runtime = runtime
        self.inner = int(p["intermediate_size"])
        gate, up = store.get(x + ".gate_proj.weight"), store.get(x + ".up_proj.weight")
        hidden = int(p["hidden_size"])
        # bfloat16 with sizes the gated kernels take: the activation is folded into the
        # product's epilogue and the stacked weight is laid out for that
        self.fused = runtime.dtype == torch.bfloat16 and self.inner % 128 == 0 and \
            ops.gated_linear_supported(hidden, 2 * self.inner)
        if self.fused:
            self.gate_up_weight = ops.interleave_gate_up(runtime.matrix(gate), runtime.matrix(up))
        else:
            self.gate_up = Linear(runtime.matrix(torch.cat([gate, up], dim=0)))
        self.down = Linear(runtime.matrix(store.get(x + ".down_proj.weight")))

    def streamed_weights(self):
        return [self.gate_up_weight if self.fused else self.gate_up.weight, self.down.weight]

    def forward(self, h):
        act = self.runtime.empty(h.shape[0], self.inner)
        if self.fused:
            ops.gated_linear(h, self.gate_up_weight, act)
        else:
            ops.silu_gate(self.gate_up.forward(h), act)
        return self.down.forward(act, partials_ok=True)


register_part("feed_forward", "gated_mlp", GatedMLP)

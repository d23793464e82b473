"""Gated feed-forward: down(act(gate(x)) * up(x)), no biases; the gate and up
products are one stacked product (reference: qwen-infer/src/model.rs:226-250,
silu(z) = z * sigmoid(z)).  The activation is a parameter of the part and of the kernels
behind it (`ops.ACTIVATIONS`); the architecture served asks for silu."""
from __future__ import annotations

import os

import torch

from ..config.spec import ConfigError
from ..kernels import ops
from ..weights.store import TensorSpec
from .base import register_part
from .linear import Linear


# TOKB200_FFN=separate runs the feed-forward of few rows as norm, gate/up and down kernels
_FUSED_STEP = os.environ.get("TOKB200_FFN", "fused") != "separate"
# Where the one-kernel feed-forward leads the separate kernels (norm, gate/up with activation, down),
# measured: up to 8 rows of a narrow stream (hidden 896: 0.69 against 0.74 ms a decoding step of 24
# layers).  With 9 to 16 rows it trails (0.91 against 0.86 ms), and so it does on a wider stream,
# where every block's own norm of all rows costs more than a launch (hidden 1,536, 32 requests with
# portions of 512 tokens: 0.63 against 0.56 s).
FUSED_ROWS = 8
FUSED_HIDDEN = 1024


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
        if p["activation"] not in ops.ACTIVATIONS:
            raise ConfigError(f"gated feed-forward knows the activations {', '.join(ops.ACTIVATIONS)}; "
                              f"found {p['activation']}")
        self.activation = p["activation"]
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

    def fused_step(self, stream, norm) -> bool:
        """For few rows in bfloat16: residual add, norm, both products and the activation
        in one kernel, straight from the stream (the norm must be one that can be folded:
        it offers `folded() -> (gain, eps)` of an RMS norm).  True when it was done; the
        stream then holds the new sum and this part's output as pending partial sums."""
        fold = getattr(norm, "folded", None)
        if not (_FUSED_STEP and self.fused and fold is not None):
            return False
        x = stream.x
        rows, hidden = x.shape
        if rows > FUSED_ROWS or hidden > FUSED_HIDDEN:
            return False
        splits = ops.ffn_small_m_splits(rows, hidden, self.inner)
        if splits == 0:
            return False
        gain, eps = fold()
        delta, stream.pending = stream.pending, None
        x_out = torch.empty_like(x)
        out = torch.empty((splits, rows, hidden), dtype=torch.float32, device=x.device)
        ops.ffn_small_m(x, x_out, delta, gain, eps, self.gate_up_weight, self.down.weight, out,
                        self.activation)
        stream.x, stream.pending = x_out, out
        return True

    def gated_operands(self):
        """(gate/up weight in the gated kernels' interleaved row order, down weight, activation)
        for a kernel that computes this feed-forward inside a larger fusion; None when the sizes
        or the precision have no such layout."""
        if not (_FUSED_STEP and self.fused):
            return None
        return self.gate_up_weight, self.down.weight, self.activation

    def streamed_weights(self):
        """What a second stream may bring into L2 ahead of a step of few rows: nothing when
        the fused kernel runs, which streams its weights itself from its first cycle."""
        if _FUSED_STEP and self.fused:
            return []
        return [self.gate_up_weight if self.fused else self.gate_up.weight, self.down.weight]

    def forward(self, h):
        act = self.runtime.empty(h.shape[0], self.inner)
        if self.fused:
            ops.gated_linear(h, self.gate_up_weight, act, self.activation)
        else:
            ops.silu_gate(self.gate_up.forward(h), act, self.activation)
        return self.down.forward(act, partials_ok=True)


register_part("feed_forward", "gated_mlp", GatedMLP)

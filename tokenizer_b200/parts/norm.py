"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * gain, statistics in float32
(reference: qwen-infer/src/model.rs:594-599, 616, 749)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.store import TensorSpec
from .base import register_part


class RMSNorm:
    @staticmethod
    def tensors(spec):
        return [TensorSpec(spec.prefix + ".weight", (spec.params["size"],), "one_plus_normal")]

    def __init__(self, spec, store, runtime):
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.runtime = runtime
        self.gain = runtime.vector(store.get(spec.prefix + ".weight"))

    def folded(self):
        """(gain, eps) for a consumer that computes this norm inside its own kernel."""
        return self.gain, self.eps

    def forward(self, x, delta=None, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = self.runtime.empty(n, self.size)
        ops.rms_norm(x, self.gain, self.eps, out, delta=delta, rows=rows)
        return out


register_part("norm", "rms_norm", RMSNorm)

"""Token embedding and output head.  The head multiplies the wanted rows, after
the final norm, by its own matrix or by the embedding it is tied to; logits are
float32 (reference: qwen-infer/src/model.rs:693-697, 750-758, 1224-1242)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.store import TensorSpec
from .base import register_part
from .linear import Linear


class TokenEmbedding:
    @staticmethod
    def tensors(spec):
        return [TensorSpec(spec.prefix + ".weight",
                           (spec.params["vocab_size"], spec.params["hidden_size"]))]

    def __init__(self, spec, store, runtime):
        self.runtime = runtime
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])
        self.table = runtime.matrix(store.get(spec.prefix + ".weight"))

    def forward(self, ids):
        x = self.runtime.empty(ids.shape[0], self.hidden, dtype=torch.float32)
        ops.embed(ids, self.table, x)
        return x


class LMHead:
    @staticmethod
    def tensors(spec):
        if spec.params.get("tied_to"):
            return []
        return [TensorSpec(spec.prefix + ".weight",
                           (spec.params["vocab_size"], spec.params["hidden_size"]))]

    def __init__(self, spec, store, runtime, tied_table=None):
        self.runtime = runtime
        if spec.params.get("tied_to"):
            if tied_table is None:
                raise ValueError("a tied head needs the embedding table")
            self.proj = Linear(tied_table)
        else:
            self.proj = Linear(runtime.matrix(store.get(spec.prefix + ".weight")))

    def forward(self, h):
        return self.proj.forward(h, out_dtype=torch.float32)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)

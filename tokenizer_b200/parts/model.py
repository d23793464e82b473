"""The generic decoder: parts assembled from a `ModelSpec`, run in the order
the spec lists.  Nothing here names an architecture."""
from __future__ import annotations

import os
from typing import List

import torch

from ..config.spec import ConfigError, ModelSpec
from ..kernels import ops
from ..weights.store import TensorSpec, WeightStore
from .base import CacheBinding, ResidualStream, Runtime, StepContext, build_part, part_class


def layer_parts(layer):
    """[(category, PartSpec)] of a layer, in the order its arrangement names them.  The
    arrangement (a registered block class) lists the names it wants and their categories in
    `PARTS`; a layer that lacks one, or brings one more, is a configuration error."""
    wanted = getattr(part_class("block", layer.block), "PARTS", None)
    if wanted is None:
        raise ConfigError(f"block {layer.block!r} does not say which parts it arranges (PARTS)")
    missing = [n for n in wanted if n not in layer.parts]
    unknown = [n for n in layer.parts if n not in wanted]
    if missing or unknown:
        raise ConfigError(f"block {layer.block!r} arranges {', '.join(wanted)}; the layer lacks "
                          f"{', '.join(missing) or 'nothing'} and brings unknown {', '.join(unknown) or 'nothing'}")
    return [(wanted[name], layer.parts[name]) for name in wanted]


def declared_tensors(spec: ModelSpec) -> List[TensorSpec]:
    """Every tensor the model's parts declare, from the spec alone."""
    out = list(part_class("embedding", spec.embedding.kind).tensors(spec.embedding))
    for layer in spec.layers:
        for category, part in layer_parts(layer):
            out += part_class(category, part.kind).tensors(part)
    out += part_class("norm", spec.final_norm.kind).tensors(spec.final_norm)
    out += part_class("head", spec.head.kind).tensors(spec.head)
    return out


# TOKB200_L2_PREFETCH=1: while a step of few rows runs a layer, a second stream brings the next
# layer's streamed weights into L2.  It gained 3 % before kernels started under programmatic
# dependent launch and asked for their weights ahead of their wait; since then it gains
# nothing (0.771 against 0.769 ms a step at batch 8) and is off unless asked for.
_PREFETCH = os.environ.get("TOKB200_L2_PREFETCH", "0") == "1"


class _Prefetcher:
    """Launches L2 prefetches on a second stream, forked from and joined to the
    stream the step runs on (which may be capturing a graph)."""

    def __init__(self, side):
        self.side, self.main, self.used = side, torch.cuda.current_stream(), False

    def fetch(self, tensors):
        self.side.wait_stream(self.main)
        with torch.cuda.stream(self.side), ops.bound_stream():
            for t in tensors:
                ops.prefetch_l2(t)
        self.used = True

    def join(self):
        if self.used:
            self.main.wait_stream(self.side)


class DecoderModel:
    def __init__(self, spec: ModelSpec, store: WeightStore, runtime: Runtime):
        spec.validate()
        ignorable = ["lm_head.weight"] if spec.head.params.get("tied_to") else []
        store.check(declared_tensors(spec), ignorable=ignorable)
        self.spec, self.runtime = spec, runtime
        self.vocab_size, self.hidden_size = spec.vocab_size, spec.hidden_size
        self.max_positions = spec.max_positions
        self.embedding = build_part("embedding", spec.embedding, store, runtime)
        self.blocks = []
        for layer in spec.layers:
            block_cls = part_class("block", layer.block)
            built = {name: build_part(category, layer.parts[name], store, runtime)
                     for name, (category, _) in zip(block_cls.PARTS, layer_parts(layer))}
            self.blocks.append(block_cls(**built))
        self.final_norm = build_part("norm", spec.final_norm, store, runtime)
        head_cls = part_class("head", spec.head.kind)
        tied = self.embedding.table if spec.head.params.get("tied_to") else None
        self.head = head_cls(spec.head, store, runtime, tied_table=tied)
        self.order = spec.order
        self._side = None
        self.scratch = ops.ScratchSpace()      # what this model's kernels use beyond inputs and outputs

    def _prefetcher(self, ctx):
        """Steps of few rows stream every weight once and wait on memory in each
        kernel; for them the next layer's weights are brought into L2 on a second
        stream while this layer runs."""
        if not _PREFETCH or self.runtime.dtype != torch.bfloat16 or ctx.n_tokens > 64:
            return None
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.runtime.device)
        return _Prefetcher(self._side)

    def parts(self):
        """Every built part of every block (the mixer first), block by block."""
        for block in self.blocks:
            for name in type(block).PARTS:
                yield name, getattr(block, name)

    def batch_annotations(self):
        """The annotations the parts want packed with every step, one per key."""
        found = {}
        for _, part in self.parts():
            for note in getattr(part, "batch_annotations", lambda: [])():
                found.setdefault(note.key, note)
        return list(found.values())

    def shape_key(self, q_lens):
        """What, beyond its sizes, decides a step's kernels: the distinct answers of the parts
        that have a say (a captured step is kept under it)."""
        kinds = []
        for _, part in self.parts():
            say = getattr(part, "shape_key", None)
            if say is not None:
                kind = say(q_lens)
                if kind not in kinds:
                    kinds.append(kind)
        return tuple(kinds)

    def graph_safe(self) -> bool:
        """Whether a step's launches depend on device-side metadata alone, so that a captured
        step can be replayed: every mixer must say so (`graph_safe = True`); any other part may
        say that it is not."""
        return all(getattr(part, "graph_safe", name != "mixer") for name, part in self.parts())

    def cache_needs(self):
        """One entry per call of the order: the need of the mixer that runs
        there, or None where the call reads an earlier call's cache."""
        needs = []
        for call in self.order:
            needs.append(None if call.cache is not None
                         else self.blocks[call.layer].mixer.cache_need())
        return needs

    def forward(self, ctx: StepContext, bindings: List[CacheBinding],
                want_rows: torch.Tensor) -> torch.Tensor:
        """Run the rows of `ctx` through every call of the order and return the
        float32 logits of `want_rows` (int32 row indices), [len(want_rows), vocab]."""
        with ops.bound_stream(), ops.scratch_scope(self.scratch):
            return self._forward(ctx, bindings, want_rows)

    def _forward(self, ctx, bindings, want_rows):
        stream = ResidualStream(self.embedding.forward(ctx.ids))
        ahead = self._prefetcher(ctx)
        for at, (call, binding) in enumerate(zip(self.order, bindings)):
            if ahead is not None and at + 1 < len(self.order):
                ahead.fetch(self.blocks[self.order[at + 1].layer].streamed_weights())
            ctx.next_block = self.blocks[self.order[at + 1].layer] if at + 1 < len(self.order) else None
            self.blocks[call.layer].forward(stream, ctx, binding)
        if ahead is not None:
            ahead.join()
        if want_rows.shape[0] == 0:
            stream.pending = None
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.runtime.device)
        stream.flush()
        h = self.final_norm.forward(stream.x, rows=want_rows)
        return self.head.forward(h)

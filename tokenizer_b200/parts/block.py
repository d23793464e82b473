"""Arrangement of a layer's parts.  Pre-norm residual: x += mixer(norm(x));
x += feed_forward(norm(x)) (reference: qwen-infer/src/model.rs:603-623).  The
adds are left pending on the stream so the next norm performs them."""
from __future__ import annotations

from .base import register_part


class PreNormResidual:
    # the parts this arrangement wants, by name, and the category each is built from; the
    # model builds them from the layer's spec and hands them over as keyword arguments
    PARTS = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm",
             "feed_forward_norm": "norm"}

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def streamed_weights(self):
        """The matrices a step with few rows reads once, in the order it reads them."""
        out = []
        for part in (self.mixer, self.feed_forward):
            out += list(getattr(part, "streamed_weights", lambda: [])())
        return out

    def layer_start_operands(self):
        """What this layer's kernels read first (the mixer's first weight, the first norm's
        gain, the mixer's bias), for the layer before to bring into L2; None when the parts
        have no such operands."""
        start = getattr(self.mixer, "start_operands", None)
        fold = getattr(self.mixer_norm, "folded", None)
        if start is None or fold is None:
            return None
        weight, bias = start()
        return weight, fold()[0], bias

    def forward(self, stream, ctx, cache):
        # a mixer may take the whole layer (both norms, itself, the feed-forward) into one kernel
        whole = getattr(self.mixer, "fused_layer", None)
        if whole is not None and whole(stream, self.mixer_norm, ctx, cache, self.feed_forward,
                                       self.feed_forward_norm):
            return
        # a mixer may take the stream as it is and fold the norm into its own kernel
        fused = getattr(self.mixer, "fused_step", None)
        delta = fused(stream, self.mixer_norm, ctx, cache) if fused is not None else None
        if delta is None:
            delta = self.mixer.forward(stream.normed(self.mixer_norm), ctx, cache)
        stream.add(delta)
        # a feed-forward may take the stream as it is and fold the norm into its own kernel
        fused = getattr(self.feed_forward, "fused_step", None)
        if fused is None or not fused(stream, self.feed_forward_norm):
            stream.add(self.feed_forward.forward(stream.normed(self.feed_forward_norm)))


register_part("block", "pre_norm_residual", PreNormResidual)

"""Grouped-query attention over the paged cache.

q = h Wq^T + bq, k = h Wk^T + bk, v = h Wv^T + bv (one fused product over the
stacked weights); q and k are rotated at their absolute positions; k (after the
rotation) and v are written into the cache pages of their request; every row
then attends to the keys of its request up to its own position (inside the
window, where the layer has one: a key is hidden when key + window < query),
scores q.k / sqrt(head_dim) with the scale applied after the product, softmax
in float32; kv head g serves query heads g*n .. (g+1)*n - 1; the merged heads go
through Wo (reference: qwen-infer/src/model.rs:262-328, 397-414, 119-129).
"""
from __future__ import annotations

import math
import os

import numpy as np
import torch

from ..config.spec import ConfigError
from ..kernels import ops
from ..weights.store import TensorSpec
from .base import BatchAnnotation, CacheNeed, KVNeed, build_part, register_part
from . import gemm_bf16
from .linear import Linear

_position_tables = {}

# Which kernel takes long prompt portions in bfloat16: the tcgen05 kernel (128-row
# tiles, scores and outputs in tensor memory; 45 us on 2,048 tokens of 14 heads) or,
# with TOKB200_ATTENTION=mma, the mma.sync kernel (64-row tiles; 73 us), which also
# takes the short portions and the head sizes the first does not.
_PROMPT_KERNEL = os.environ.get("TOKB200_ATTENTION", "tcgen05")
# TOKB200_QKV_NORM=separate keeps the norm in front of the projection of few rows a kernel of its own
# TOKB200_QKV_ROPE=fused folds rotation and cache write of many rows into the tcgen05 product's
# epilogue.  With one tile a block the longer epilogue is not hidden behind other tiles, and it
# costs what the separate kernel costs (3.27 against 3.26 ms for 2,048 tokens), so it is off
# unless asked for.
_FUSED_QKV = os.environ.get("TOKB200_QKV_ROPE", "separate") == "fused"
_FUSED_NORM = os.environ.get("TOKB200_QKV_NORM", "fused") != "separate"
# TOKB200_LAYER=fused runs a decoding step's layer (up to 32 rows) as ONE kernel instead of four
# (projection, attention, output projection, feed-forward).  It is correct and off by default:
# measured at 36 us a layer against 27 us for the four kernels (8 rows, Qwen2.5-0.5B sizes),
# because its phases run one after the other behind barriers over all blocks, each a chain of
# two or three trips to L2, while the four kernels overlap their heads and tails.  The
# switches that take the norm or the feed-forward out of their fusions turn it off as well.
_FUSED_LAYER = os.environ.get("TOKB200_LAYER", "separate") == "fused" and _FUSED_NORM


class RowTiles(BatchAnnotation):
    """The step's rows cut into tiles of up to `rows` consecutive rows of one request, as the
    prompt-attention kernels take them: int32 [tiles, 2] = (first row, rows), the tile that
    walks the most keys first (the kernels place blocks in that order, so the longest work
    starts first).  Unused tiles of a padded step have no rows.  With `long_only`, requests
    that bring a single token get no tile when others bring more (their rows are `SingleRows`',
    served by the decoding kernel: a tile of one row would walk its keys at a tile's cost)."""

    def __init__(self, rows: int, long_only: bool = False):
        self.rows = rows
        self.long_only = long_only
        self.key = f"row_tiles_{rows}" + ("_long" if long_only else "")

    def capacity(self, n_tokens, n_requests):
        return 2 * (n_tokens // self.rows + n_requests)

    def fill(self, out, first_rows, counts, starts, padded):
        n = len(counts)
        if self.long_only and n and int(counts.max()) > 1:
            keep = counts > 1
            first_rows, counts, starts = first_rows[keep], counts[keep], starts[keep]
            n = len(counts)
        if n and int(counts.max()) == 1:
            # one tile of one row a request: a stable order, as a sort of tuples gives
            order = np.argsort(-starts, kind="stable")
            out[0:2 * n:2] = first_rows[order]
            out[1:2 * n:2] = 1
            made = n
        else:
            tiles = []    # (last position + 1: the keys the tile walks, first row, rows)
            for first_row, count, start in zip(first_rows.tolist(), counts.tolist(), starts.tolist()):
                for first in range(0, count, self.rows):
                    here = min(self.rows, count - first)
                    tiles.append((start + first + here, first_row + first, here))
            tiles.sort(key=lambda item: -item[0])
            for at, (_, first_row, here) in enumerate(tiles):
                out[2 * at] = first_row
                out[2 * at + 1] = here
            made = len(tiles)
        return len(out) // 2 if padded else made

    def view(self, words):
        return words.view(-1, 2)


class SingleRows(BatchAnnotation):
    """The rows of requests that bring exactly one token, when the step also brings portions
    of others: int32 [requests], row indices, -1 where there is none.  A step of single tokens
    alone has none (all of its rows go to the decoding kernel anyway)."""

    key = "single_rows"

    def capacity(self, n_tokens, n_requests):
        return n_requests

    def fill(self, out, first_rows, counts, starts, padded):
        out[:] = -1
        made = 0
        if len(counts) and int(counts.max()) > 1:
            rows = first_rows[counts == 1]
            out[:len(rows)] = rows
            made = len(rows)
        # a captured step keeps the launch for as many rows as it has requests, but only a step
        # that has such rows at all: steps of portions alone are captured without it (their key
        # differs, see Attention.shape_key)
        return (len(out) if made else 0) if padded else made


# the tiles of the two prompt kernels: 64 rows (mma.sync) and 128 rows (tcgen05), for all
# requests and for those alone that bring more than one token
_TILES = RowTiles(ops.PREFILL_TILE_ROWS)
_WIDE_TILES = RowTiles(ops.WIDE_TILE_ROWS)
_LONG_TILES = RowTiles(ops.PREFILL_TILE_ROWS, long_only=True)
_LONG_WIDE_TILES = RowTiles(ops.WIDE_TILE_ROWS, long_only=True)
_SINGLES = SingleRows()
# TOKB200_MIXED=tiles sends the single-token rows of a mixed step through the kernels for portions
_SPLIT_MIXED = os.environ.get("TOKB200_MIXED", "split") != "tiles"
# portions from this length on go to the tcgen05 kernel (shorter ones would leave most of a
# 128-row tile empty)
_WIDE_FROM = 96


class GQAttention:
    graph_safe = True   # launches depend on device-side metadata only

    def batch_annotations(self):
        return [_TILES, _WIDE_TILES, _LONG_TILES, _LONG_WIDE_TILES, _SINGLES]

    def shape_key(self, q_lens):
        """Which attention kernel a step of these portion lengths gets (part of the key under
        which the engine keeps a captured step)."""
        longest = max(q_lens) if q_lens else 0
        if longest == 1:
            return "single"
        kind = "wide" if longest >= _WIDE_FROM else "tiles"
        # portions with single tokens beside them launch the decoding kernel too
        return kind + "+1" if min(q_lens) == 1 else kind

    @staticmethod
    def tensors(spec):
        p, x = spec.params, spec.prefix
        q_out, kv_out = p["num_heads"] * p["head_dim"], p["num_kv_heads"] * p["head_dim"]
        out = [
            TensorSpec(x + ".q_proj.weight", (q_out, p["hidden_size"])),
            TensorSpec(x + ".k_proj.weight", (kv_out, p["hidden_size"])),
            TensorSpec(x + ".v_proj.weight", (kv_out, p["hidden_size"])),
            TensorSpec(x + ".o_proj.weight", (p["hidden_size"], q_out)),
        ]
        if p.get("qkv_bias"):
            out += [TensorSpec(x + ".q_proj.bias", (q_out,)),
                    TensorSpec(x + ".k_proj.bias", (kv_out,)),
                    TensorSpec(x + ".v_proj.bias", (kv_out,))]
        if p.get("out_bias"):
            out.append(TensorSpec(x + ".o_proj.bias", (p["hidden_size"],)))
        return out

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        self.runtime = runtime
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.window = p.get("window")
        if self.nh % self.nkv:
            raise ConfigError(f"{self.nh} query heads is not a multiple of {self.nkv} kv heads")
        if self.d % 2:
            raise ConfigError(f"head size {self.d} must be even")
        self.scale = 1.0 / math.sqrt(float(self.d))
        # one stacked product for q, k and v
        w_qkv = torch.cat([store.get(x + f".{n}_proj.weight") for n in "qkv"], dim=0)
        self.qkv = Linear(runtime.matrix(w_qkv))
        self.qkv_bias = None
        if p.get("qkv_bias"):
            self.qkv_bias = runtime.vector(
                torch.cat([store.get(x + f".{n}_proj.bias").to(torch.float32) for n in "qkv"]))
        self.out = Linear(
            runtime.matrix(store.get(x + ".o_proj.weight")),
            runtime.vector(store.get(x + ".o_proj.bias")) if p.get("out_bias") else None)
        # layers with the same position constants share one table
        pos_spec = p["position"]
        key = (pos_spec.kind, tuple(sorted(pos_spec.params.items())), str(runtime.device))
        if key not in _position_tables:
            _position_tables[key] = build_part("position", pos_spec, store, runtime)
        self.position = _position_tables[key]
        if self.position.rotary_dim > self.d:
            raise ConfigError("the rotary width exceeds the head size")

    def cache_need(self):
        return CacheNeed(kv=KVNeed(self.nkv, self.d, self.window))

    def streamed_weights(self):
        return [self.qkv.weight, self.out.weight]

    def start_operands(self):
        """(first weight, its bias): what this mixer's first kernel reads."""
        return self.qkv.weight, self.qkv_bias

    def fused_layer(self, stream, norm, ctx, cache, feed_forward, feed_forward_norm) -> bool:
        """For a step of few rows of one token each in bfloat16: the WHOLE pre-norm layer in one
        kernel (both norms, this attention, a gated feed-forward), straight from the stream.
        The norms must offer `folded() -> (gain, eps)` of an RMS norm and the feed-forward
        `gated_operands() -> (interleaved gate/up weight, down weight, activation)`.  True when it
        was done: the stream then holds the sum after the attention, and the feed-forward's output
        as pending partial sums.  False: the block runs the parts one by one."""
        fold, fold2 = getattr(norm, "folded", None), getattr(feed_forward_norm, "folded", None)
        operands = getattr(feed_forward, "gated_operands", None)
        x = stream.x
        if not (_FUSED_LAYER and fold is not None and fold2 is not None and operands is not None and
                self.runtime.dtype == torch.bfloat16 and ctx.max_q_len == 1 and self.out.bias is None and
                self.position.rotary_dim == self.d and cache.k_pool is not None):
            return False
        gated = operands()
        if gated is None:
            return False
        w_gate_up, w_down, activation = gated
        down_splits, _ = ops.layer_small_m_splits(x.shape[0], self.hidden, w_down.shape[1], self.nh, self.nkv, self.d)
        if down_splits == 0:
            return False
        (gain1, eps1), (gain2, eps2) = fold(), fold2()
        group = ctx.groups[cache.group]
        delta, stream.pending = stream.pending, None
        x_mid, x_out = torch.empty_like(x), torch.empty_like(x)
        out = torch.empty((down_splits,) + tuple(x.shape), dtype=torch.float32, device=x.device)
        ahead = getattr(ctx.next_block, "layer_start_operands", None)
        ops.layer_small_m(x, delta, x_mid, x_out, out, gain1, eps1, self.qkv.weight, self.qkv_bias, ctx.pos,
                          group.slots, ctx.row_req, group.block_table, self.position.cos, self.position.sin,
                          cache.k_pool, cache.v_pool, cache.writes, self.out.weight, gain2, eps2, w_gate_up,
                          w_down, self.nh, self.nkv, self.d, group.page_size, self.window, self.scale, activation,
                          next_layer=ahead() if ahead is not None else None)
        stream.x, stream.pending = x_out, out
        return True

    def fused_step(self, stream, norm, ctx, cache):
        """For few rows in bfloat16: the residual add and the norm in front are computed by
        the projection kernel itself, straight from the stream (the norm must offer
        `folded() -> (gain, eps)` of an RMS norm).  Returns this part's output, or None when
        the sizes are not taken (the block then norms and calls `forward`)."""
        fold = getattr(norm, "folded", None)
        x = stream.x
        if not (_FUSED_NORM and fold is not None and self.runtime.dtype == torch.bfloat16 and
                ops.qkv_norm_rope_small_m_supported(x.shape[0], self.hidden, self.d,
                                                    self.position.rotary_dim)):
            return None
        gain, eps = fold()
        group = ctx.groups[cache.group]
        delta, stream.pending = stream.pending, None
        x_out = torch.empty_like(x)
        q = self.runtime.empty(ctx.n_tokens, self.nh * self.d)
        ops.qkv_norm_rope_small_m(
            x, x_out, delta, gain, eps, self.qkv.weight, self.qkv_bias, ctx.pos,
            group.slots if cache.writes else None, self.position.cos, self.position.sin, q,
            cache.k_pool if cache.writes else None, cache.v_pool if cache.writes else None,
            self.nh, self.nkv, self.d)
        stream.x = x_out
        mixed = self.runtime.empty(ctx.n_tokens, self.nh * self.d)
        self.attend(q, mixed, ctx, group, cache)
        return self.out.forward(mixed, partials_ok=True)

    def forward(self, h, ctx, cache):
        q = self.runtime.empty(ctx.n_tokens, self.nh * self.d)
        group = ctx.groups[cache.group]
        if h.dtype == torch.bfloat16 and ops.qkv_rope_small_m_supported(
                h.shape[0], self.hidden, self.d, self.position.rotary_dim, self.qkv.out_features):
            # few rows: projection, bias, rotation and cache write in one kernel
            ops.qkv_rope_small_m(
                h, self.qkv.weight, self.qkv_bias, ctx.pos, group.slots if cache.writes else None,
                self.position.cos, self.position.sin, q,
                cache.k_pool if cache.writes else None, cache.v_pool if cache.writes else None,
                self.nh, self.nkv, self.d)
            mixed = self.runtime.empty(ctx.n_tokens, self.nh * self.d)
            self.attend(q, mixed, ctx, group, cache)
            return self.out.forward(mixed, partials_ok=True)
        if h.dtype == torch.bfloat16 and _FUSED_QKV and \
                gemm_bf16.choose_tile_k_splits(h.shape[0], self.qkv.out_features, self.hidden) == 1 and \
                gemm_bf16.use_tcgen05(h.shape[0], self.qkv.out_features, self.hidden) and \
                ops.gemm_qkv_rope_supported(self.hidden, self.nh, self.nkv, self.d, self.position.rotary_dim):
            # many rows: the tcgen05 product with bias, rotation and cache write in its epilogue
            ops.gemm_qkv_rope(
                h, self.qkv.weight, self.qkv_bias, ctx.pos, group.slots if cache.writes else None,
                self.position.cos, self.position.sin, q,
                cache.k_pool if cache.writes else None, cache.v_pool if cache.writes else None,
                self.nh, self.nkv, self.d)
            mixed = self.runtime.empty(ctx.n_tokens, self.nh * self.d)
            self.attend(q, mixed, ctx, group, cache)
            return self.out.forward(mixed, partials_ok=True)
        # in bfloat16 with a whole-head rotation the product may come as partial sums over k
        # (a few dozen rows and a narrow matrix fill the device only that way)
        sums_ok = h.dtype == torch.bfloat16 and self.position.rotary_dim == self.d and self.d % 16 == 0
        qkv = self.qkv.forward(h, partials_ok=sums_ok)
        ops.rope_store(
            qkv, self.qkv_bias, ctx.pos, group.slots if cache.writes else None,
            self.position.cos, self.position.sin, q,
            cache.k_pool if cache.writes else None, cache.v_pool if cache.writes else None,
            self.nh, self.nkv, self.d, self.position.rotary_dim)
        mixed = self.runtime.empty(ctx.n_tokens, self.nh * self.d)
        self.attend(q, mixed, ctx, group, cache)
        return self.out.forward(mixed, partials_ok=True)

    def attend(self, q, out, ctx, group, cache):
        """Choose the kernel by precision and by the shape of the batch."""
        if q.dtype == torch.bfloat16 and ctx.max_q_len == 1 and \
                ops.decode_attention_supported(self.nh, self.nkv, self.d):
            ops.decode_attention(
                q, cache.k_pool, cache.v_pool, out, group.block_table, ctx.row_req, ctx.pos,
                self.nh, self.nkv, self.d, group.page_size, self.window, self.scale)
            return
        wide, tiles = ctx.views.get(_WIDE_TILES.key), ctx.views.get(_TILES.key)
        singles = ctx.views.get(_SINGLES.key)
        if _SPLIT_MIXED and q.dtype == torch.bfloat16 and singles is not None and singles[1] > 0 and \
                ops.decode_attention_supported(self.nh, self.nkv, self.d) and \
                ctx.views.get(_LONG_WIDE_TILES.key) is not None and ctx.views.get(_LONG_TILES.key) is not None:
            # a step of portions AND single tokens: the single-token rows go to the decoding kernel
            # (keys split over blocks, the group's heads as one tile), the portions to theirs
            ops.decode_attention(
                q, cache.k_pool, cache.v_pool, out, group.block_table, ctx.row_req, ctx.pos,
                self.nh, self.nkv, self.d, group.page_size, self.window, self.scale, rows=singles[0])
            wide, tiles = ctx.views[_LONG_WIDE_TILES.key], ctx.views[_LONG_TILES.key]
        if _PROMPT_KERNEL == "tcgen05" and q.dtype == torch.bfloat16 and \
                wide is not None and ctx.max_q_len >= _WIDE_FROM and \
                ops.attention_tcgen05_supported(self.nh, self.nkv, self.d):
            # long portions on the tcgen05 kernel (128-row tiles, scores in tensor memory)
            ops.attention_tcgen05(
                q, cache.k_pool, cache.v_pool, out, group.block_table, ctx.row_req, ctx.pos,
                wide[0], wide[1], self.nh, self.nkv, self.d, group.page_size,
                self.window, self.scale)
            return
        if q.dtype == torch.bfloat16 and tiles is not None and \
                ops.prefill_attention_supported(self.nh, self.nkv, self.d):
            ops.prefill_attention(
                q, cache.k_pool, cache.v_pool, out, group.block_table, ctx.row_req, ctx.pos,
                tiles[0], tiles[1], self.nh, self.nkv, self.d, group.page_size,
                self.window, self.scale)
            return
        ops.paged_attention_generic(
            q, cache.k_pool, cache.v_pool, out, group.block_table, ctx.row_req, ctx.pos,
            self.nh, self.nkv, self.d, group.page_size, self.window, self.scale)


register_part("mixer", "gqa_attention", GQAttention)

"""Plain, slow, whole-sequence Qwen2 decoder in 32-bit on the CPU.

This file is the oracle of the test-suite.  It is written from the formulas of
the reference's `qwen-infer/src/model.rs` and `qwen-infer/src/sample.rs`
(each function cites file:line) and shares no code with the engine under
`tokenizer_b200/`: it has its own safetensors access (the `safetensors`
package), its own config reading, no cache, no batching, one function per
part.  The reference itself is Rust on candle and can be neither imported nor
compiled where these tests run, so this implementation rests on the formulas.
"""
from __future__ import annotations

import json
import math
import os

import torch


# --------------------------------------------------------------------------- #
# loading
# --------------------------------------------------------------------------- #
def load_folder(folder):
    """config.json as a dict and every tensor as float32 (model.rs:776-786:
    the file is mapped and each tensor is converted to f32 on read)."""
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    raw = load_file(os.path.join(folder, "model.safetensors"))
    weights = {name: t.to(torch.float32) for name, t in raw.items()}
    return cfg, weights


def head_dim_of(cfg):
    """model.rs:739: head_dim = hidden_size / num_attention_heads (a
    `head_dim` key, where config.json gives one, takes its place)."""
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


# --------------------------------------------------------------------------- #
# parts
# --------------------------------------------------------------------------- #
def embed(ids, table):
    """model.rs:837-838: x[t, :] = E[ids[t], :]."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def rms_norm(x, gain, eps):
    """model.rs:594,616 (candle rms_norm): y = x / sqrt(mean(x^2) + eps) * w."""
    x = x.to(torch.float32)
    mean_sq = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(mean_sq + eps) * gain


def linear(x, weight, bias=None):
    """model.rs:289-291: y = x W^T (+ b), weights stored (out, in)."""
    y = x @ weight.t()
    if bias is not None:
        y = y + bias
    return y


def rope_tables(theta, dim, n_positions):
    """model.rs:145-164: inv_freq_i = 1/theta^(i/dim) for even i, computed in
    f64 and stored f32; angle = f32(position) * inv_freq in f32; cos and sin of
    that, shape (positions, dim/2)."""
    inv_freq = torch.tensor(
        [float(1.0 / (float(theta) ** (i / dim))) for i in range(0, dim, 2)],
        dtype=torch.float64,
    ).to(torch.float32)
    positions = torch.arange(n_positions, dtype=torch.float32).reshape(-1, 1)
    freqs = positions * inv_freq.reshape(1, -1)
    return torch.cos(freqs), torch.sin(freqs)


def rope_apply(x, cos, sin):
    """model.rs:166-172 (candle rotary_emb::rope, half-split form): for a head
    vector x, out[i] = x[i] cos - x[i+d/2] sin, out[i+d/2] = x[i+d/2] cos +
    x[i] sin.  x is (heads, seq, d); cos, sin are (seq, d/2) for the absolute
    positions of the rows."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def mask_value(query, key, window):
    """model.rs:119-129: -inf if key > query; with a window W also -inf if
    key + W < query; else 0."""
    if key > query:
        return -math.inf
    if window is not None and key + window < query:
        return -math.inf
    return 0.0


def attention_mask(seq, window):
    """model.rs:923-940 for a whole sequence (query and key origin equal): the matrix of
    `mask_value(query, key, window)`, filled by comparisons over whole index arrays so that
    sequences of thousands of tokens stay affordable (tests/test_plain.py compares it with
    the entry-by-entry rule)."""
    query = torch.arange(seq).reshape(-1, 1)
    key = torch.arange(seq).reshape(1, -1)
    hidden = key > query
    if window is not None:
        hidden = hidden | (key + int(window) < query)
    return torch.zeros((seq, seq), dtype=torch.float32).masked_fill(hidden, -math.inf)


def window_for_layer(cfg, index):
    """model.rs:909-915: the window holds for layer i only if
    use_sliding_window and i >= max_window_layers."""
    if cfg.get("use_sliding_window") and index >= cfg["max_window_layers"]:
        return int(cfg["sliding_window"])
    return None


def attention(x, w, prefix, cfg, cos, sin, window):
    """model.rs:280-328: q/k/v projections with bias, head split, RoPE on q and
    k, GQA by repeating each kv head over its group (model.rs:566-580), scores
    = q k^T * (1/sqrt(d)) applied after the product, additive mask, softmax
    over keys, mix, merge heads, o projection without bias."""
    seq = x.shape[0]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = head_dim_of(cfg)
    q = linear(x, w[prefix + "q_proj.weight"], w[prefix + "q_proj.bias"])
    k = linear(x, w[prefix + "k_proj.weight"], w[prefix + "k_proj.bias"])
    v = linear(x, w[prefix + "v_proj.weight"], w[prefix + "v_proj.bias"])
    q = q.reshape(seq, nh, d).transpose(0, 1)
    k = k.reshape(seq, nkv, d).transpose(0, 1)
    v = v.reshape(seq, nkv, d).transpose(0, 1)
    q = rope_apply(q, cos[:seq], sin[:seq])
    k = rope_apply(k, cos[:seq], sin[:seq])
    groups = nh // nkv
    k = k.repeat_interleave(groups, dim=0)
    v = v.repeat_interleave(groups, dim=0)
    scale = 1.0 / math.sqrt(float(d))
    scores = (q @ k.transpose(1, 2)) * scale
    scores = scores + attention_mask(seq, window)
    weights = torch.softmax(scores, dim=-1)
    mixed = weights @ v
    merged = mixed.transpose(0, 1).reshape(seq, nh * d)
    return linear(merged, w[prefix + "o_proj.weight"])


def swiglu_mlp(x, w, prefix):
    """model.rs:245-249: down(silu(gate(x)) * up(x)), silu(z) = z sigmoid(z),
    no biases."""
    gate = linear(x, w[prefix + "gate_proj.weight"])
    up = linear(x, w[prefix + "up_proj.weight"])
    return linear(gate * torch.sigmoid(gate) * up, w[prefix + "down_proj.weight"])


def decoder_layer(x, w, index, cfg, cos, sin):
    """model.rs:603-623: norm -> attention -> add -> norm -> mlp -> add."""
    p = f"model.layers.{index}."
    eps = cfg["rms_norm_eps"]
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    x = attention(h, w, p + "self_attn.", cfg, cos, sin, window_for_layer(cfg, index)) + x
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    return swiglu_mlp(h, w, p + "mlp.") + x


def all_logits(cfg, w, ids, rows=None):
    """Logits at every position of `ids`, (seq, vocab), by a full recompute
    (model.rs:832-848 keeps the last row only; every row is the same product).
    Head: model.rs:1224-1242, tied to the embedding or `lm_head.weight`.  With `rows`
    (positions), only those rows go through the final norm and the head: (len(rows), vocab)."""
    seq = len(ids)
    if seq == 0 or seq > cfg["max_position_embeddings"]:
        raise ValueError("positions exceed max_position_embeddings")
    cos, sin = rope_tables(cfg["rope_theta"], head_dim_of(cfg), seq)
    x = embed(ids, w["model.embed_tokens.weight"])
    for index in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, index, cfg, cos, sin)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    h = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(h, head)


# --------------------------------------------------------------------------- #
# sampling
# --------------------------------------------------------------------------- #
def greedy_token(logits):
    """sample.rs:44-57: argmax with strict `>`, so ties keep the lower id."""
    best_at, best = 0, -math.inf
    for index, value in enumerate(logits.tolist()):
        if value > best:
            best, best_at = value, index
    return best_at


def sample_intervals(logits, temperature, top_p):
    """sample.rs:91-124: weights exp((l - max)/T); candidates ordered by logit
    descending, ties by lower index; the kept set is the shortest prefix whose
    cumulative probability reaches top_p (at least one; top_p >= 1 keeps all).
    Returns the kept ids in walking order and their weights."""
    values = torch.as_tensor(logits, dtype=torch.float32)
    weight = torch.exp((values - values.max()) / temperature)
    order = sorted(range(len(values)), key=lambda i: (-float(values[i]), i))
    if top_p >= 1.0:
        keep = len(order)
    else:
        total = float(weight.sum())
        cumulative, keep = 0.0, 1
        for k, index in enumerate(order):
            cumulative += float(weight[index]) / total
            keep = k + 1
            if cumulative >= top_p:
                break
    kept = order[:keep]
    return kept, [float(weight[i]) for i in kept]


def sample_token(logits, temperature, top_p, u):
    """sample.rs:66-137 with the uniform draw `u` in [0,1) given by the caller:
    threshold = u * kept_sum, walk the kept ids in order, return the first
    whose mass exceeds what is left of the threshold."""
    if temperature == 0.0:
        return greedy_token(torch.as_tensor(logits))
    kept, mass = sample_intervals(logits, temperature, top_p)
    threshold = u * sum(mass)
    for index, m in zip(kept, mass):
        if threshold < m:
            return index
        threshold -= m
    return kept[-1]


def greedy_generate(cfg, w, prompt, n_new):
    """lib.rs:120-133 (`greedy_tokens`): full recompute, append the argmax."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        token = greedy_token(all_logits(cfg, w, ids)[-1])
        out.append(token)
        ids.append(token)
    return out

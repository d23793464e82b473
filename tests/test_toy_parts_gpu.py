"""Parts of other kinds, defined here, are registered, built and stepped without a
change to the framework's files: a feed-forward with routing (top-1 of three experts,
weighted by the router's probability) and another position encoding (rotary angles
of interpolated positions), in a toy architecture that chooses them layer by layer
beside the framework's own parts and whose order names a layer twice."""
import os

import pytest
import torch

import plain_qwen2 as plain
from tiny import random_ids

pytestmark = pytest.mark.gpu

HIDDEN, VOCAB, INNER, EXPERTS, FACTOR = 64, 150, 48, 3, 4.0
ORDER = (0, 1, 2, 1)          # layer 1 runs twice, each call with a cache of its own


class TopOneExperts:
    """delta = p_e * down_e(silu(up_e h)), e = argmax of the router's logits (32-bit),
    p = softmax of the logits.  Dense over the experts and masked, so that a captured
    step holds no choice made on the host."""
    graph_safe = True

    @staticmethod
    def tensors(spec):
        from tokenizer_b200.weights import TensorSpec
        p, x = spec.params, spec.prefix
        out = [TensorSpec(x + ".router.weight", (p["experts"], p["hidden_size"]), "normal", 3.0)]
        for e in range(p["experts"]):
            out.append(TensorSpec(x + f".experts.{e}.up.weight", (p["inner"], p["hidden_size"]), "normal", 0.2))
            out.append(TensorSpec(x + f".experts.{e}.down.weight", (p["hidden_size"], p["inner"]), "normal", 0.2))
        return out

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        self.router = store.get(x + ".router.weight").to(runtime.device, torch.float32)
        self.up = [runtime.matrix(store.get(x + f".experts.{e}.up.weight")) for e in range(p["experts"])]
        self.down = [runtime.matrix(store.get(x + f".experts.{e}.down.weight")) for e in range(p["experts"])]

    def forward(self, h):
        logits = h.float() @ self.router.t()
        prob = torch.softmax(logits, dim=-1)
        chosen = logits.argmax(dim=-1)
        out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
        for e, (up, down) in enumerate(zip(self.up, self.down)):
            inner = torch.nn.functional.silu((h @ up.t()).float()).to(h.dtype)
            weight = torch.where(chosen == e, prob[:, e], torch.zeros_like(prob[:, e]))
            out += (inner @ down.t()).float() * weight[:, None]
        return out.to(h.dtype)


class InterpolatedRotary:
    """Rotary tables of positions divided by a factor (what the mixer reads: `rotary_dim`,
    `cos`, `sin` of `max_positions` rows)."""

    @staticmethod
    def tensors(spec):
        return []

    def __init__(self, spec, store, runtime):
        p = spec.params
        self.rotary_dim, self.max_positions = int(p["rotary_dim"]), int(p["max_positions"])
        self.cos, self.sin = (t.to(runtime.device) for t in toy_tables(p["theta"], self.rotary_dim,
                                                                      self.max_positions, p["factor"]))


def toy_tables(theta, dim, n, factor):
    inv_freq = torch.tensor([1.0 / (float(theta) ** (i / dim)) for i in range(0, dim, 2)],
                            dtype=torch.float64).to(torch.float32)
    angles = (torch.arange(n, dtype=torch.float32) / factor)[:, None] * inv_freq[None, :]
    return torch.cos(angles).contiguous(), torch.sin(angles).contiguous()


class ToyConfig:
    def __init__(self, raw):
        self.raw = raw

    @classmethod
    def from_dict(cls, raw):
        return cls(dict(raw))

    def to_dict(self):
        return dict(self.raw)

    def model_spec(self):
        from tokenizer_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec
        norm = PartSpec("rms_norm", {"size": HIDDEN, "eps": 1e-5})
        rope = PartSpec("rope_half_split", {"theta": 1e4, "rotary_dim": 16, "max_positions": 256})
        toy_rope = PartSpec("toy_rope_interpolated", {"theta": 500.0, "rotary_dim": 16,
                                                      "max_positions": 256, "factor": FACTOR})
        layers = []
        for i in range(3):
            p = f"toy.layers.{i}"
            mixer = PartSpec("gqa_attention", {
                "hidden_size": HIDDEN, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "qkv_bias": True,
                "out_bias": False, "window": None, "position": rope if i == 1 else toy_rope}, p + ".self_attn")
            if i == 1:
                ff = PartSpec("gated_mlp", {"hidden_size": HIDDEN, "intermediate_size": 128,
                                            "activation": "silu"}, p + ".mlp")
            else:
                ff = PartSpec("toy_top1_experts", {"hidden_size": HIDDEN, "inner": INNER,
                                                   "experts": EXPERTS}, p + ".moe")
            layers.append(LayerSpec("pre_norm_residual", mixer, ff,
                                    norm.with_prefix(p + ".norm1"), norm.with_prefix(p + ".norm2")))
        return ModelSpec("ToyPartsForTest", VOCAB, HIDDEN, 256,
                         PartSpec("token_embedding", {"vocab_size": VOCAB, "hidden_size": HIDDEN}, "toy.embed"),
                         tuple(layers), tuple(LayerCall(i) for i in ORDER), norm.with_prefix("toy.norm"),
                         PartSpec("lm_head", {"vocab_size": VOCAB, "hidden_size": HIDDEN, "tied_to": None}, "toy.head"))


def toy_reference(folder, ids):
    """Whole sequence, no cache; returns the logits and, per row, the smallest lead of the
    chosen expert over the runner-up (rows with a thin lead may go the other way in bfloat16)."""
    from safetensors.torch import load_file
    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    cfg = {"num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16}
    tables = {True: plain.rope_tables(1e4, 16, len(ids)), False: toy_tables(500.0, 16, len(ids), FACTOR)}
    x = plain.embed(ids, w["toy.embed.weight"])
    lead = torch.full((len(ids),), float("inf"))
    for i in ORDER:
        p = f"toy.layers.{i}."
        cos, sin = tables[i == 1]
        x = plain.attention(plain.rms_norm(x, w[p + "norm1.weight"], 1e-5), w, p + "self_attn.", cfg, cos, sin, None) + x
        h = plain.rms_norm(x, w[p + "norm2.weight"], 1e-5)
        if i == 1:
            x = plain.swiglu_mlp(h, w, p + "mlp.") + x
            continue
        logits = h @ w[p + "moe.router.weight"].t()
        top = torch.topk(logits, 2, dim=-1).values
        lead = torch.minimum(lead, top[:, 0] - top[:, 1])
        prob, chosen = torch.softmax(logits, -1), logits.argmax(-1)
        delta = torch.zeros_like(x)
        for t in range(len(ids)):
            e = int(chosen[t])
            inner = torch.nn.functional.silu(h[t] @ w[p + f"moe.experts.{e}.up.weight"].t())
            delta[t] = prob[t, e] * (inner @ w[p + f"moe.experts.{e}.down.weight"].t())
        x = delta + x
    logits = plain.linear(plain.rms_norm(x, w["toy.norm.weight"], 1e-5), w["toy.head.weight"])
    return logits, lead


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_another_position_encoding(dtype, tmp_path):
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import Engine, StepEntry
    from tokenizer_b200.parts import register_part

    register_part("feed_forward", "toy_top1_experts", TopOneExperts)
    register_part("position", "toy_rope_interpolated", InterpolatedRotary)
    tb.register_architecture("ToyPartsForTest", ToyConfig)
    config = ToyConfig({"architectures": ["ToyPartsForTest"]})
    folder = tb.write_random_model(str(tmp_path / "toy"), config, seed=23,
                                   scale={r"\.(q|k)_proj\.weight": 6.0, "embed|head": 5.0})
    engine = Engine.from_folder(folder, dtype=dtype, num_pages=24, page_size=8, max_requests=2)
    # four calls of the order keep keys: one group, four caches (layer 1 twice)
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].calls == [0, 1, 2, 3]
    requests = {"a": random_ids(50, VOCAB, 4), "b": random_ids(37, VOCAB, 5)}
    live = {n: engine.cache.open(n) for n in requests}
    done, got = {n: 0 for n in requests}, {n: [] for n in requests}
    plan = [{"a": 9, "b": 30}, {"a": 1, "b": 1}, {"a": 1, "b": 1}, {"a": 1, "b": 1}, {"a": 38, "b": 4}]
    for portion in plan:          # portions, then single tokens (a captured step, replayed), then a mix
        entries = []
        for n, count in portion.items():
            engine.cache.reserve(live[n], count)
            entries.append(StepEntry(live[n], requests[n][done[n]:done[n] + count], list(range(count))))
        logits = engine.step(entries).float().cpu()
        at = 0
        for n, count in portion.items():
            got[n].append(logits[at:at + count])
            at += count
            done[n] += count
    checked = 0
    for n, ids in requests.items():
        want, lead = toy_reference(folder, ids)
        result = torch.cat(got[n])
        assert result.shape == want.shape
        bound = 1e-4 if dtype == "float32" else 2e-2 * float(want.abs().max())
        # a row's keys come from earlier rows: one thin lead spoils the rows after it too
        sure = torch.cumprod((lead > (1e-4 if dtype == "float32" else 0.25)).long(), 0).bool()
        err = (result - want).abs().max(dim=1).values
        assert float(err[sure].max()) <= bound, f"{n}: first wrong row {int((err > bound).nonzero()[0])}"
        checked += int(sure.sum())
    assert checked >= 30

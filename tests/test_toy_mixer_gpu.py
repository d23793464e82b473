"""A mixer with state of its own, defined here, is registered, built and stepped
without a change to the framework's files: a toy architecture whose layers
alternate between the toy mixer (a running mean over the request's rows, kept
in a per-request state slot) and the framework's attention."""
import json
import os

import pytest
import torch

import plain_qwen2 as plain
from tiny import random_ids

pytestmark = pytest.mark.gpu

HIDDEN, VOCAB, LAYERS = 48, 200, 4


class RunningMeanMixer:
    """out[t] = (mean of the request's rows 0..t) W^T.  State per request: the
    sum of the rows so far and their count."""

    @staticmethod
    def tensors(spec):
        from tokenizer_b200.weights import TensorSpec
        n = spec.params["hidden_size"]
        return [TensorSpec(spec.prefix + ".mix.weight", (n, n), "normal", 0.2)]

    def __init__(self, spec, store, runtime):
        self.n = int(spec.params["hidden_size"])
        self.runtime = runtime
        self.weight = store.get(spec.prefix + ".mix.weight").to(runtime.device, torch.float32)

    def cache_need(self):
        from tokenizer_b200.parts import CacheNeed, StateNeed
        return CacheNeed(state=StateNeed((self.n + 1,)))

    def forward(self, h, ctx, cache):
        out = torch.empty_like(h)
        at = 0
        for count, slot in zip(ctx.q_lens, ctx.state_slots):
            state = cache.state[slot]
            rows = h[at:at + count].float()
            sums = state[:self.n] + torch.cumsum(rows, 0)
            counts = state[self.n] + torch.arange(1, count + 1, device=h.device, dtype=torch.float32)
            out[at:at + count] = ((sums / counts[:, None]) @ self.weight.t()).to(h.dtype)
            state[:self.n] = sums[-1]
            state[self.n] = counts[-1]
            at += count
        return out


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
        position = PartSpec("rope_half_split", {"theta": 1e4, "rotary_dim": 16, "max_positions": 256})
        layers = []
        for i in range(LAYERS):
            p = f"toy.layers.{i}"
            if i % 2 == 0:
                mixer = PartSpec("toy_running_mean", {"hidden_size": HIDDEN}, p + ".mean")
            else:
                mixer = PartSpec("gqa_attention", {
                    "hidden_size": HIDDEN, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16,
                    "qkv_bias": True, "out_bias": False, "window": None, "position": position},
                    p + ".self_attn")
            layers.append(LayerSpec(
                "pre_norm_residual", mixer,
                PartSpec("gated_mlp", {"hidden_size": HIDDEN, "intermediate_size": 80,
                                       "activation": "silu"}, p + ".mlp"),
                norm.with_prefix(p + ".norm1"), norm.with_prefix(p + ".norm2")))
        return ModelSpec("ToyStateForTest", VOCAB, HIDDEN, 256,
                         PartSpec("token_embedding", {"vocab_size": VOCAB, "hidden_size": HIDDEN}, "toy.embed"),
                         tuple(layers), tuple(LayerCall(i) for i in range(LAYERS)),
                         norm.with_prefix("toy.norm"),
                         PartSpec("lm_head", {"vocab_size": VOCAB, "hidden_size": HIDDEN, "tied_to": None}, "toy.head"))


def toy_reference(folder, ids):
    from safetensors.torch import load_file
    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    cfg = {"num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16}
    cos, sin = plain.rope_tables(1e4, 16, len(ids))
    x = plain.embed(ids, w["toy.embed.weight"])
    for i in range(LAYERS):
        p = f"toy.layers.{i}."
        h = plain.rms_norm(x, w[p + "norm1.weight"], 1e-5)
        if i % 2 == 0:
            mean = torch.cumsum(h, 0) / torch.arange(1, len(ids) + 1, dtype=torch.float32)[:, None]
            x = mean @ w[p + "mean.mix.weight"].t() + x
        else:
            x = plain.attention(h, w, p + "self_attn.", cfg, cos, sin, None) + x
        h = plain.rms_norm(x, w[p + "norm2.weight"], 1e-5)
        x = plain.swiglu_mlp(h, w, p + "mlp.") + x
    return plain.linear(plain.rms_norm(x, w["toy.norm.weight"], 1e-5), w["toy.head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_mixer_with_state_is_registered_built_and_stepped(dtype, tmp_path):
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import Engine, StepEntry
    from tokenizer_b200.parts import register_part

    register_part("mixer", "toy_running_mean", RunningMeanMixer)
    tb.register_architecture("ToyStateForTest", ToyConfig)
    config = ToyConfig({"architectures": ["ToyStateForTest"]})
    folder = tb.write_random_model(str(tmp_path / "toy"), config, seed=11,
                                   scale={r"\.(q|k)_proj\.weight": 8.0, "embed|head": 5.0})
    assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["ToyStateForTest"]
    engine = Engine.from_folder(folder, dtype=dtype, num_pages=12, page_size=8, max_requests=3)
    # two layers keep keys (one group), two keep state (two arenas); pages only for the former
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].calls == [1, 3]
    assert sorted(engine.cache.states) == [0, 2]
    requests = {"a": random_ids(40, VOCAB, 1), "b": random_ids(33, VOCAB, 2), "c": random_ids(21, VOCAB, 3)}
    want = {n: toy_reference(folder, ids) for n, ids in requests.items()}
    live, done, got = {}, {n: 0 for n in requests}, {n: [] for n in requests}
    plan = [{"a": 7, "b": 2}, {"a": 1, "b": 30}, {"a": 20, "b": 1}, {"a": 12}]
    for portion in plan:
        entries = []
        for n, count in portion.items():
            if n not in live:
                live[n] = engine.cache.open(n)
            engine.cache.reserve(live[n], count)
            entries.append(StepEntry(live[n], requests[n][done[n]:done[n] + count], list(range(count))))
        logits = engine.step(entries).cpu()
        at = 0
        for n, count in portion.items():
            got[n].append(logits[at:at + count])
            at += count
            done[n] += count
    # "b" ends; "c" takes its state slot, which must start from zero again
    slot_b = live["b"].state_slot
    engine.cache.close(live.pop("b"))
    live["c"] = engine.cache.open("c")
    assert live["c"].state_slot == slot_b
    engine.cache.reserve(live["c"], 21)
    got["c"].append(engine.step([StepEntry(live["c"], requests["c"], list(range(21)))]).cpu())
    for n in requests:
        result = torch.cat(got[n])
        assert result.shape == want[n].shape
        scale = float(want[n].abs().max())
        bound = 1e-4 if dtype == "float32" else 2e-2 * scale
        err = (result - want[n]).abs().max(dim=1).values
        assert float(err.max()) <= bound, f"{n}: first wrong row {int((err > bound).nonzero()[0])}"

"""Another arrangement of a layer's parts, defined here and registered without a change to the
framework's files: a block with a THIRD norm (the mixer's output is normed before it joins the
residual sum) and its feed-forward beside, not behind, the mixer.  The layers of the toy
architecture alternate between it and the framework's pre-norm block; one layer's mixer is the
stateful toy mixer, so the model is not replayed from graphs and its device-side decoding
steps are launched one by one."""
import os

import pytest
import torch

import plain_qwen2 as plain
from test_toy_mixer_gpu import RunningMeanMixer
from tiny import random_ids

pytestmark = pytest.mark.gpu

HIDDEN, VOCAB, LAYERS, HEAD = 64, 150, 3, 16


class SandwichParallel:
    """x += post_norm(mixer(norm(x))) + feed_forward(ff_norm(x)): both branches read the same
    residual sum.  The arranged parts arrive as keyword arguments under the names of PARTS."""

    PARTS = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm",
             "feed_forward_norm": "norm", "mixer_post_norm": "norm"}

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, mixer_post_norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.mixer_post_norm = mixer_post_norm

    def streamed_weights(self):
        return []

    def forward(self, stream, ctx, cache):
        x = stream.flush()
        mixed = self.mixer.forward(self.mixer_norm.forward(x), ctx, cache)
        mixed = self.mixer_post_norm.forward(self._as_stream(mixed))
        fed = self.feed_forward.forward(self.feed_forward_norm.forward(x))
        if fed.dim() == 3:               # partial sums over k: add them up
            fed = fed.sum(0)
        stream.add((mixed.float() + fed.float()).to(mixed.dtype))

    @staticmethod
    def _as_stream(t):
        if t.dim() == 3:
            t = t.sum(0)
        return t.float().contiguous()


class ToyBlockConfig:
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
        position = PartSpec("rope_half_split", {"theta": 1e4, "rotary_dim": HEAD, "max_positions": 256})
        layers = []
        for i in range(LAYERS):
            p = f"toy.layers.{i}"
            if i == 1:
                mixer = PartSpec("toy_running_mean", {"hidden_size": HIDDEN}, p + ".mean")
            else:
                mixer = PartSpec("gqa_attention", {
                    "hidden_size": HIDDEN, "num_heads": 4, "num_kv_heads": 2, "head_dim": HEAD,
                    "qkv_bias": True, "out_bias": False, "window": None, "position": position},
                    p + ".self_attn")
            ff = PartSpec("gated_mlp", {"hidden_size": HIDDEN, "intermediate_size": 128,
                                        "activation": "silu"}, p + ".mlp")
            if i % 2 == 0:
                layers.append(LayerSpec("toy_sandwich_parallel", mixer=mixer, feed_forward=ff,
                                        mixer_norm=norm.with_prefix(p + ".norm1"),
                                        feed_forward_norm=norm.with_prefix(p + ".norm2"),
                                        mixer_post_norm=norm.with_prefix(p + ".norm3")))
            else:
                layers.append(LayerSpec("pre_norm_residual", mixer, ff,
                                        norm.with_prefix(p + ".norm1"), norm.with_prefix(p + ".norm2")))
        return ModelSpec("ToyBlockForTest", VOCAB, HIDDEN, 256,
                         PartSpec("token_embedding", {"vocab_size": VOCAB, "hidden_size": HIDDEN}, "toy.embed"),
                         tuple(layers), tuple(LayerCall(i) for i in range(LAYERS)),
                         norm.with_prefix("toy.norm"),
                         PartSpec("lm_head", {"vocab_size": VOCAB, "hidden_size": HIDDEN, "tied_to": None}, "toy.head"))


def toy_reference(folder, ids):
    from safetensors.torch import load_file
    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    cfg = {"num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": HEAD}
    cos, sin = plain.rope_tables(1e4, HEAD, len(ids))
    x = plain.embed(ids, w["toy.embed.weight"])
    for i in range(LAYERS):
        p = f"toy.layers.{i}."
        h = plain.rms_norm(x, w[p + "norm1.weight"], 1e-5)
        if i == 1:
            mean = torch.cumsum(h, 0) / torch.arange(1, len(ids) + 1, dtype=torch.float32)[:, None]
            mixed = mean @ w[p + "mean.mix.weight"].t()
        else:
            mixed = plain.attention(h, w, p + "self_attn.", cfg, cos, sin, None)
        if i % 2 == 0:
            fed = plain.swiglu_mlp(plain.rms_norm(x, w[p + "norm2.weight"], 1e-5), w, p + "mlp.")
            x = x + plain.rms_norm(mixed, w[p + "norm3.weight"], 1e-5) + fed
        else:
            x = x + mixed
            x = x + plain.swiglu_mlp(plain.rms_norm(x, w[p + "norm2.weight"], 1e-5), w, p + "mlp.")
    return plain.linear(plain.rms_norm(x, w["toy.norm.weight"], 1e-5), w["toy.head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_block_with_a_third_norm_is_registered_built_and_stepped(dtype, tmp_path):
    import tokenizer_b200 as tb
    from tokenizer_b200.config.spec import ConfigError
    from tokenizer_b200.engine import Engine, StepEntry
    from tokenizer_b200.parts import register_part

    register_part("mixer", "toy_running_mean", RunningMeanMixer)
    register_part("block", "toy_sandwich_parallel", SandwichParallel)
    tb.register_architecture("ToyBlockForTest", ToyBlockConfig)
    config = ToyBlockConfig({"architectures": ["ToyBlockForTest"]})
    folder = tb.write_random_model(str(tmp_path / "toy"), config, seed=13,
                                   scale={r"\.(q|k)_proj\.weight": 8.0, "embed|head": 5.0})
    engine = Engine.from_folder(folder, dtype=dtype, num_pages=24, page_size=8, max_requests=2)
    assert not engine.use_graphs                  # the toy mixer's launches depend on host-side values
    ids = random_ids(60, VOCAB, 7)
    want = toy_reference(folder, ids)
    cache = engine.cache.open("a")
    got, done = [], 0
    for count in (9, 2, 30, 1, 1):
        engine.cache.reserve(cache, count)
        got.append(engine.step([StepEntry(cache, ids[done:done + count], list(range(count)))]).cpu())
        done += count
    result = torch.cat(got)
    bound = 1e-4 if dtype == "float32" else 2e-2 * float(want.abs().max())
    err = (result - want[:done]).abs().max(dim=1).values
    assert float(err.max()) <= bound, f"first wrong row {int((err > bound).nonzero()[0])}"
    # device-side steps of a model that is not replayed from graphs: launched one by one, with the
    # state moving on; each id is the best of the plain logits of the sequence so far
    drawn = engine.decode_steps([StepEntry(cache, [ids[done]])], 6)
    sequence = ids[:done + 1] + [row[0] for row in drawn]
    logits = toy_reference(folder, sequence[:-1])
    for k, row in enumerate(drawn):
        lead = logits[done + k]
        assert float(lead.max() - lead[row[0]]) <= 2 * bound, f"device-side step {k}"
    assert cache.length == done + 6
    # a layer that lacks a part its block arranges is refused by name
    from tokenizer_b200.config import LayerSpec
    from tokenizer_b200.parts.model import layer_parts
    broken = LayerSpec("toy_sandwich_parallel", *[config.model_spec().layers[0].parts[n] for n in
                                                  ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm")])
    with pytest.raises(ConfigError, match="mixer_post_norm"):
        layer_parts(broken)

"""Each part of the model alone, built from a PartSpec with sizes of its own,
against the plain implementation's function for the same part; and the run
order as data: a layer named twice, a layer that reads another layer's cache."""
import dataclasses
import math

import pytest
import torch

import plain_qwen2 as plain
from tiny import random_ids

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def runtime(dtype):
    from tokenizer_b200.parts import Runtime
    return Runtime(DEV, dtype)


def store_for(specs, seed=0, scale=None):
    from tokenizer_b200.weights import WeightStore, random_tensors
    return WeightStore(random_tensors(specs, seed, scale))


def tol(dtype):
    return dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from tokenizer_b200.config import PartSpec
    from tokenizer_b200.parts import build_part, part_class
    spec = PartSpec("rms_norm", {"size": 70, "eps": 1e-3}, "n")
    store = store_for(part_class("norm", "rms_norm").tensors(spec))
    norm = build_part("norm", spec, store, runtime(dtype))
    x = torch.randn(5, 70, generator=torch.Generator().manual_seed(1)).to(DEV)
    want = plain.rms_norm(x.cpu(), store.get("n.weight").float(), 1e-3)
    assert torch.allclose(norm.forward(x).float().cpu(), want, **tol(dtype))


def test_position_part_matches_the_tables():
    from tokenizer_b200.config import PartSpec
    from tokenizer_b200.parts import build_part
    for theta, dim in ((10000.0, 16), (1e6, 64), (5e5, 48)):
        part = build_part("position", PartSpec("rope_half_split", {
            "theta": theta, "rotary_dim": dim, "max_positions": 3000}), None, runtime(torch.float32))
        cos, sin = plain.rope_tables(theta, dim, 3000)
        # float32 cosines of angles up to 3000 rad: the angle's own rounding is ~2e-4
        assert torch.allclose(part.cos.cpu(), cos, atol=5e-6) and torch.allclose(part.sin.cpu(), sin, atol=5e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from tokenizer_b200.config import PartSpec
    from tokenizer_b200.parts import build_part, part_class
    spec = PartSpec("gated_mlp", {"hidden_size": 72, "intermediate_size": 200, "activation": "silu"}, "mlp")
    store = store_for(part_class("feed_forward", "gated_mlp").tensors(spec), scale={"": 5.0})
    part = build_part("feed_forward", spec, store, runtime(dtype))
    h = torch.randn(6, 72, generator=torch.Generator().manual_seed(2)).to(dtype)
    weights = {k: store.get(k).float() for k in store.names()}
    want = plain.swiglu_mlp(h.float(), weights, "mlp.")
    got = part.forward(h.to(DEV)).float().cpu()
    assert torch.allclose(got, want, **tol(dtype)), float((got - want).abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [6, 150])
def test_feed_forward_part_with_another_activation(dtype, rows):
    """The activation is the part's parameter: the same part with a tanh-gelu gate (sizes the
    gated kernels take, so that in bfloat16 the activation runs in their epilogues)."""
    from tokenizer_b200.config import PartSpec
    from tokenizer_b200.config.spec import ConfigError
    from tokenizer_b200.parts import build_part, part_class
    params = {"hidden_size": 64, "intermediate_size": 256, "activation": "gelu_pytorch_tanh"}
    spec = PartSpec("gated_mlp", params, "mlp")
    store = store_for(part_class("feed_forward", "gated_mlp").tensors(spec), scale={"": 5.0})
    part = build_part("feed_forward", spec, store, runtime(dtype))
    h = torch.randn(rows, 64, generator=torch.Generator().manual_seed(3)).to(dtype)
    w = {k: store.get(k).float() for k in store.names()}
    g, u = h.float() @ w["mlp.gate_proj.weight"].t(), h.float() @ w["mlp.up_proj.weight"].t()
    act = 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    want = (act * u) @ w["mlp.down_proj.weight"].t()
    got = part.forward(h.to(DEV)).float()
    got = (got.sum(0) if got.dim() == 3 else got).cpu()
    assert torch.allclose(got, want, **tol(dtype)), float((got - want).abs().max())
    with pytest.raises(ConfigError, match="activations"):
        build_part("feed_forward", PartSpec("gated_mlp", dict(params, activation="swish-ish"), "mlp"), store,
                   runtime(dtype))


def small_model_pieces(dtype, window=None, nh=6, nkv=3, d=16, hidden=40):
    from tokenizer_b200.config import PartSpec
    position = PartSpec("rope_half_split", {"theta": 1e4, "rotary_dim": d, "max_positions": 256})
    mixer = PartSpec("gqa_attention", {
        "hidden_size": hidden, "num_heads": nh, "num_kv_heads": nkv, "head_dim": d, "qkv_bias": True,
        "out_bias": False, "window": window, "position": position}, "attn")
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": d, "hidden_size": hidden}
    return mixer, cfg


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_over_portions(dtype, window):
    """The mixer alone: two requests, fed in portions; every row must equal
    the plain whole-sequence attention of its request."""
    from tokenizer_b200.cache.device import DeviceCache
    from tokenizer_b200.engine.batch import BatchBuilder, StepEntry
    from tokenizer_b200.parts import build_part, part_class
    from tokenizer_b200.config.spec import LayerCall
    spec, cfg = small_model_pieces(dtype, window)
    store = store_for(part_class("mixer", "gqa_attention").tensors(spec), seed=3,
                      scale={r"(q|k)_proj\.weight": 10.0, r"v_proj|o_proj": 5.0})
    rt = runtime(dtype)
    mixer = build_part("mixer", spec, store, rt)
    cache = DeviceCache([mixer.cache_need()], num_pages=16, page_size=4, max_requests=2, runtime=rt)
    binding = cache.bindings([LayerCall(0)])[0]
    builder = BatchBuilder(cache, 10, 256, DEV, mixer.batch_annotations())
    g = torch.Generator().manual_seed(4)
    hs = {"a": torch.randn(23, 40, generator=g).to(dtype), "b": torch.randn(14, 40, generator=g).to(dtype)}
    weights = {k: store.get(k).float() for k in store.names()}
    cos, sin = plain.rope_tables(1e4, 16, 64)
    want = {n: plain.attention(h.float(), weights, "attn.", cfg, cos, sin, window) for n, h in hs.items()}
    live = {n: cache.open(n) for n in hs}
    done = {n: 0 for n in hs}
    for portion in ({"a": 5, "b": 2}, {"a": 1}, {"a": 9, "b": 11}, {"b": 1, "a": 8}):
        entries, rows = [], []
        for n, count in portion.items():
            cache.reserve(live[n], count)
            entries.append(StepEntry(live[n], [0] * count, []))
            rows.append(hs[n][done[n]:done[n] + count])
        ctx, _, _ = builder.build(entries)
        out = mixer.forward(torch.cat(rows).to(DEV).contiguous(), ctx, binding).float().cpu()
        at = 0
        for n, count in portion.items():
            ref = want[n][done[n]:done[n] + count]
            assert torch.allclose(out[at:at + count], ref, **tol(dtype)), (n, done[n], float((out[at:at + count] - ref).abs().max()))
            cache.commit(live[n], count)
            done[n] += count
            at += count
    assert done == {"a": 23, "b": 14}


def plain_with_order(cfg, w, ids, order, reads):
    """The plain parts run in an arbitrary order of layers; `reads[i]` names the
    earlier call whose keys and values call i uses instead of its own."""
    seq = len(ids)
    d = plain.head_dim_of(cfg)
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    cos, sin = plain.rope_tables(cfg["rope_theta"], d, seq)
    x = plain.embed(ids, w["model.embed_tokens.weight"])
    kept = {}
    for at, layer in enumerate(order):
        p = f"model.layers.{layer}."
        h = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        a = p + "self_attn."
        q = plain.linear(h, w[a + "q_proj.weight"], w[a + "q_proj.bias"]).reshape(seq, nh, d).transpose(0, 1)
        q = plain.rope_apply(q, cos, sin)
        if reads[at] is None:
            k = plain.linear(h, w[a + "k_proj.weight"], w[a + "k_proj.bias"]).reshape(seq, nkv, d).transpose(0, 1)
            v = plain.linear(h, w[a + "v_proj.weight"], w[a + "v_proj.bias"]).reshape(seq, nkv, d).transpose(0, 1)
            kept[at] = (plain.rope_apply(k, cos, sin), v)
        k, v = kept[at if reads[at] is None else reads[at]]
        k, v = k.repeat_interleave(nh // nkv, 0), v.repeat_interleave(nh // nkv, 0)
        s = (q @ k.transpose(1, 2)) / math.sqrt(d) + plain.attention_mask(seq, None)
        mixed = (torch.softmax(s, -1) @ v).transpose(0, 1).reshape(seq, nh * d)
        x = plain.linear(mixed, w[a + "o_proj.weight"]) + x
        h = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        x = plain.swiglu_mlp(h, w, p + "mlp.") + x
    h = plain.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    return plain.linear(h, w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_order_is_data_a_layer_twice_and_a_shared_cache(dtype, tmp_path):
    from tiny import TINY
    from tokenizer_b200 import write_random_model
    from tokenizer_b200.config.spec import LayerCall
    from tokenizer_b200.engine import Engine, StepEntry
    from tokenizer_b200.parts import DecoderModel
    from tokenizer_b200.weights import WeightStore
    config = TINY["a"]()[0]
    folder = write_random_model(str(tmp_path / "m"), config, 7,
                                scale={r"\.(q|k)_proj\.weight": 8.0, "embed_tokens": 5.0})
    # layer 0, layer 1, layer 0 again (a cache of its own), layer 1 reading the cache of call 1
    order = (LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache=1))
    spec = dataclasses.replace(config.model_spec(), order=order)
    model = DecoderModel(spec, WeightStore.from_folder(folder), runtime(dtype))
    assert [n is None for n in model.cache_needs()] == [False, False, False, True]
    engine = Engine(model, num_pages=8, page_size=16)
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].calls == [0, 1, 2]
    ids = random_ids(50, config.vocab_size, 5)
    cfg, w = plain.load_folder(folder)
    want = plain_with_order(cfg, w, ids, [0, 1, 0, 1], [None, None, None, 1])
    cache = engine.cache.open("r")
    got = []
    for lo, hi in ((0, 20), (20, 22), (22, 49), (49, 50)):
        engine.cache.reserve(cache, hi - lo)
        got.append(engine.step([StepEntry(cache, ids[lo:hi], list(range(hi - lo)))]).cpu())
    got = torch.cat(got)
    scale = float(want.abs().max())
    bound = 1e-4 if dtype == torch.float32 else 2e-2 * scale
    assert float((got - want).abs().max()) <= bound
    # and it is not the plain order: the result differs from running the layers once
    assert float((plain.all_logits(cfg, w, ids) - want).abs().max()) > 0.02 * scale

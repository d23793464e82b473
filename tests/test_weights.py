"""Weights by name: stored precision, the one error that lists everything,
random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

from tokenizer_b200.parts import declared_tensors
from tokenizer_b200.weights import (WeightError, WeightStore, read_safetensors, write_random_model,
                                    write_safetensors)
from tiny import TINY


def test_random_folder_is_a_function_of_config_and_seed(tmp_path):
    config = TINY["b"]()[0]
    a = write_random_model(str(tmp_path / "a"), config, 5)
    b = write_random_model(str(tmp_path / "b"), config, 5)
    c = write_random_model(str(tmp_path / "c"), config, 6)
    ta, tb, tc = (read_safetensors(os.path.join(f, "model.safetensors")) for f in (a, b, c))
    assert sorted(ta) == sorted(tb) == sorted(tc)
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert any(not torch.equal(ta[k], tc[k]) for k in ta)
    assert json.load(open(os.path.join(a, "config.json")))["architectures"] == ["Qwen2ForCausalLM"]
    # names and shapes are the Hugging Face ones
    assert ta["model.layers.2.self_attn.k_proj.weight"].shape == (32, 96)
    assert ta["model.layers.0.self_attn.q_proj.bias"].shape == (96,)
    assert ta["model.layers.1.mlp.down_proj.weight"].shape == (96, 256)
    assert ta["lm_head.weight"].shape == (1000, 96)
    assert "lm_head.weight" not in read_safetensors(
        os.path.join(write_random_model(str(tmp_path / "t"), TINY["a"]()[0], 0), "model.safetensors"))
    # statistics of the init: N(0, 0.02) and gains 1 + N(0, 0.02), stored in bfloat16
    w = ta["model.layers.0.mlp.gate_proj.weight"]
    assert w.dtype == torch.bfloat16
    assert abs(float(w.float().std()) - 0.02) < 2e-3 and abs(float(w.float().mean())) < 1e-3
    g = ta["model.norm.weight"].float()
    assert abs(float(g.mean()) - 1.0) < 2e-2 and float(g.std()) > 5e-3


def test_stored_precision_is_kept(tmp_path):
    path = str(tmp_path / "m.safetensors")
    write_safetensors(path, {
        "bf": torch.randn(3, 4).to(torch.bfloat16), "f32": torch.randn(5),
        "f16": torch.randn(2, 2).to(torch.float16), "table": torch.arange(6, dtype=torch.int64)})
    store = WeightStore(read_safetensors(path), path)
    assert store.get("bf").dtype == torch.bfloat16
    assert store.get("f32").dtype == torch.float32        # 32-bit stays 32-bit
    assert store.get("f16").dtype == torch.bfloat16
    assert store.get("table").dtype == torch.int32         # integer tables are int32
    assert store.get("table").tolist() == list(range(6))
    with pytest.raises(WeightError, match="no tensor nothere"):
        store.get("nothere")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config = TINY["a"]()[0]
    folder = write_random_model(str(tmp_path / "m"), config, 0)
    path = os.path.join(folder, "model.safetensors")
    tensors = dict(read_safetensors(path))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(65, dtype=torch.bfloat16)
    write_safetensors(path, tensors)
    store = WeightStore.from_folder(folder)
    with pytest.raises(WeightError) as err:
        store.check(declared_tensors(config.model_spec()))
    text = str(err.value)
    assert "missing (2): model.layers.1.mlp.up_proj.weight, model.norm.weight" in text
    assert "unexpected (1): model.layers.0.self_attn.rotary.inv_freq" in text
    assert "wrong shape: model.layers.0.self_attn.q_proj.bias is [65], the model needs [64]" in text


def test_a_stored_head_beside_a_tied_one_is_tolerated(tmp_path):
    config = TINY["a"]()[0]
    folder = write_random_model(str(tmp_path / "m"), config, 0)
    path = os.path.join(folder, "model.safetensors")
    tensors = dict(read_safetensors(path))
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(path, tensors)
    WeightStore.from_folder(folder).check(declared_tensors(config.model_spec()),
                                          ignorable=["lm_head.weight"])


def test_malformed_files(tmp_path):
    p = tmp_path / "model.safetensors"
    with pytest.raises(WeightError, match="does not exist"):
        read_safetensors(str(p))
    p.write_bytes(b"abc")
    with pytest.raises(WeightError, match="too short"):
        read_safetensors(str(p))
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightError, match="exceeds"):
        read_safetensors(str(p))
    header = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 8)
    with pytest.raises(WeightError, match="x has 8 bytes"):
        read_safetensors(str(p))


def test_a_folder_of_several_files_with_an_index(tmp_path):
    """`model.safetensors.index.json` names the file of each tensor; the store reads them all and
    the check sees one set of names.  A tensor in two files, a file outside the folder and an
    index without a map are refused."""
    config = TINY["a"]()[0]
    whole = tmp_path / "whole"
    write_random_model(str(whole), config, 3)
    tensors = read_safetensors(str(whole / "model.safetensors"))
    names = sorted(tensors)
    parts = tmp_path / "parts"
    parts.mkdir()
    cut = len(names) // 2
    files = {"model-00001-of-00002.safetensors": names[:cut], "model-00002-of-00002.safetensors": names[cut:]}
    for file, held in files.items():
        write_safetensors(str(parts / file), {n: tensors[n] for n in held})
    index = {"metadata": {}, "weight_map": {n: f for f, held in files.items() for n in held}}
    (parts / "model.safetensors.index.json").write_text(json.dumps(index))
    store = WeightStore.from_folder(str(parts))
    assert store.names() == names
    assert all(torch.equal(store.get(n), tensors[n]) for n in names)
    store.check(declared_tensors(config.model_spec()))
    # the same tensor in a second file
    write_safetensors(str(parts / "model-00002-of-00002.safetensors"),
                      {n: tensors[n] for n in names[cut - 1:]})
    with pytest.raises(WeightError, match="more than one file"):
        WeightStore.from_folder(str(parts))
    index["weight_map"][names[0]] = "../whole/model.safetensors"
    (parts / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(WeightError, match="not a file name inside the folder"):
        WeightStore.from_folder(str(parts))
    (parts / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}}))
    with pytest.raises(WeightError, match="weight_map"):
        WeightStore.from_folder(str(parts))


def test_seeded_tensors_stand_in_for_a_file():
    """Random weights without a folder: each tensor is a function of (seed, name), drawn when
    asked for; the store checks shapes without drawing anything."""
    import torch
    from tokenizer_b200.weights import SeededTensors, TensorSpec, WeightError, WeightStore
    specs = [TensorSpec("a.weight", (40, 30)), TensorSpec("n.weight", (30,), "one_plus_normal"),
             TensorSpec("z.bias", (5,), "zeros")]
    source = SeededTensors(specs, seed=5)
    drawn = []
    original = SeededTensors.__getitem__
    SeededTensors.__getitem__ = lambda self, name: drawn.append(name) or original(self, name)
    try:
        store = WeightStore(source)
        store.check(specs)
        assert drawn == []
        with pytest.raises(WeightError, match="wrong shape: a.weight"):
            store.check([TensorSpec("a.weight", (40, 31))] + specs[1:])
        a = store.get("a.weight")
    finally:
        SeededTensors.__getitem__ = original
    assert a.dtype == torch.bfloat16 and tuple(a.shape) == (40, 30)
    assert torch.equal(a, store.get("a.weight"))
    assert not torch.equal(a, WeightStore(SeededTensors(specs, seed=6)).get("a.weight"))
    assert abs(float(a.float().std()) - 0.02) < 0.004
    assert abs(float(store.get("n.weight").float().mean()) - 1.0) < 0.02
    assert float(store.get("z.bias").abs().sum()) == 0.0

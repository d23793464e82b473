"""Configuration and registry (no GPU)."""
import json

import pytest

from tokenizer_b200.config import (ConfigError, Qwen2Config, config_from_dict, load_config,
                                   register_architecture, registered_architectures)
from tiny import TINY


def raw_a():
    return TINY["a"]()[0].to_dict()


def test_round_trip_and_sizes():
    for name in TINY:
        config = TINY[name]()[0]
        again = config_from_dict(json.loads(json.dumps(config.to_dict())))
        assert again == config
        spec = config.model_spec()
        assert len(spec.layers) == config.num_hidden_layers
        assert [c.layer for c in spec.order] == list(range(config.num_hidden_layers))
        assert spec.vocab_size == config.vocab_size


def test_head_dim_defaults_to_width_over_heads():
    raw = raw_a()
    del raw["head_dim"]
    assert config_from_dict(raw).head_dim == raw["hidden_size"] // raw["num_attention_heads"]
    raw["head_dim"] = 48
    assert config_from_dict(raw).head_dim == 48


def test_every_reference_key_is_required():
    for key in ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                "num_attention_heads", "num_key_value_heads", "max_position_embeddings",
                "sliding_window", "max_window_layers", "tie_word_embeddings", "rope_theta",
                "rms_norm_eps", "use_sliding_window", "hidden_act"]:
        raw = raw_a()
        del raw[key]
        with pytest.raises(ConfigError, match=key):
            config_from_dict(raw)


def test_unknown_keys_are_ignored():
    raw = raw_a()
    raw["some_future_key"] = 7
    assert config_from_dict(raw) == TINY["a"]()[0]


@pytest.mark.parametrize("change, message", [
    ({"hidden_act": "gelu"}, "silu"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"max_position_embeddings": 0}, "max_position_embeddings"),
    ({"vocab_size": "512"}, "integer"),
    ({"tie_word_embeddings": 1}, "true or false"),
    ({"head_dim": 15}, "even"),
])
def test_validation(change, message):
    raw = raw_a()
    raw.update(change)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


def test_width_must_divide_into_heads_without_head_dim():
    raw = raw_a()
    del raw["head_dim"]
    raw["hidden_size"] = 66
    with pytest.raises(ConfigError, match="does not divide"):
        config_from_dict(raw)


def test_window_applies_from_max_window_layers():
    config = TINY["c"]()[0]
    windows = [layer.mixer.params["window"] for layer in config.model_spec().layers]
    assert windows == [None, None, 24, 24]
    assert all(l.mixer.params["window"] is None for l in TINY["a"]()[0].model_spec().layers)


def test_registry_names_unknown_architecture(tmp_path):
    raw = raw_a()
    raw["architectures"] = ["NoSuchModel"]
    with pytest.raises(ConfigError, match="NoSuchModel.*Qwen2ForCausalLM"):
        config_from_dict(raw)
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({"vocab_size": 3})
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not JSON"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="does not exist"):
        load_config(str(tmp_path / "nowhere"))


def test_registering_another_architecture():
    class Other:
        @classmethod
        def from_dict(cls, raw):
            return cls()

        def to_dict(self):
            return {"architectures": ["OtherForTest"]}

        def model_spec(self):
            return None

    register_architecture("OtherForTest", Other)
    assert "OtherForTest" in registered_architectures()
    assert isinstance(config_from_dict({"architectures": ["OtherForTest"]}), Other)
    with pytest.raises(TypeError):
        register_architecture("Broken", object)


def test_order_validation():
    from tokenizer_b200.config import LayerCall
    import dataclasses
    spec = TINY["a"]()[0].model_spec()
    twice = dataclasses.replace(spec, order=(LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache=1)))
    twice.validate()
    with pytest.raises(ConfigError, match="does not run before"):
        dataclasses.replace(spec, order=(LayerCall(0, cache=1), LayerCall(1))).validate()
    with pytest.raises(ConfigError, match="names layer"):
        dataclasses.replace(spec, order=(LayerCall(5),)).validate()

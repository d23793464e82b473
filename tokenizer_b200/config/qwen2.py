"""Typed configuration of the Qwen2 dense decoder (`Qwen2ForCausalLM`).

The keys are the ones the reference's `Config` reads (qwen-infer/src/model.rs:
25-42) and, like there, all of them are required and unknown keys are ignored;
`head_dim` is read where config.json has it and is hidden_size /
num_attention_heads otherwise (model.rs:739).  Validation follows
model.rs:714-738.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

from .registry import register_architecture
from .spec import (ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec, as_bool, as_float,
                   as_int, require_keys)

ARCHITECTURE = "Qwen2ForCausalLM"

_REQUIRED = [
    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "num_key_value_heads", "max_position_embeddings",
    "sliding_window", "max_window_layers", "tie_word_embeddings", "rope_theta",
    "rms_norm_eps", "use_sliding_window", "hidden_act",
]


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    sliding_window: Optional[int]
    max_window_layers: int
    use_sliding_window: bool
    tie_word_embeddings: bool
    rope_theta: float
    rms_norm_eps: float
    hidden_act: str

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen2Config":
        require_keys(raw, _REQUIRED, ARCHITECTURE)
        use_window = as_bool(raw, "use_sliding_window")
        if raw["sliding_window"] is None and not use_window:
            window = None
        else:
            window = as_int(raw, "sliding_window", 1)
        heads = as_int(raw, "num_attention_heads", 1)
        hidden = as_int(raw, "hidden_size", 1)
        if raw.get("head_dim") is not None:
            head_dim = as_int(raw, "head_dim", 1)
        else:
            if hidden % heads:
                raise ConfigError(f"hidden_size {hidden} does not divide into {heads} heads")
            head_dim = hidden // heads
        cfg = cls(
            vocab_size=as_int(raw, "vocab_size", 1),
            hidden_size=hidden,
            intermediate_size=as_int(raw, "intermediate_size", 1),
            num_hidden_layers=as_int(raw, "num_hidden_layers", 1),
            num_attention_heads=heads,
            num_key_value_heads=as_int(raw, "num_key_value_heads", 1),
            head_dim=head_dim,
            max_position_embeddings=as_int(raw, "max_position_embeddings", 1),
            sliding_window=window,
            max_window_layers=as_int(raw, "max_window_layers", 0),
            use_sliding_window=use_window,
            tie_word_embeddings=as_bool(raw, "tie_word_embeddings"),
            rope_theta=as_float(raw, "rope_theta"),
            rms_norm_eps=as_float(raw, "rms_norm_eps"),
            hidden_act=raw["hidden_act"],
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.hidden_act != "silu":
            raise ConfigError(f"expected hidden_act silu, found {self.hidden_act}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"{self.num_attention_heads} query heads is not a multiple of "
                f"{self.num_key_value_heads} kv heads")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for the rotary encoding")
        if self.rope_theta <= 0 or self.rms_norm_eps < 0:
            raise ConfigError("rope_theta must be positive and rms_norm_eps not negative")

    def to_dict(self) -> Dict[str, Any]:
        return {
            "architectures": [ARCHITECTURE],
            "model_type": "qwen2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "use_sliding_window": self.use_sliding_window,
            "tie_word_embeddings": self.tie_word_embeddings,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "hidden_act": self.hidden_act,
            "torch_dtype": "bfloat16",
        }

    def window_for_layer(self, index: int) -> Optional[int]:
        """model.rs:909-915."""
        if self.use_sliding_window and index >= self.max_window_layers:
            return self.sliding_window
        return None

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rms_norm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        position = PartSpec("rope_half_split", {
            "theta": self.rope_theta, "rotary_dim": self.head_dim,
            "max_positions": self.max_position_embeddings})
        layers = []
        for index in range(self.num_hidden_layers):
            prefix = f"model.layers.{index}"
            mixer = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "qkv_bias": True,
                "out_bias": False,
                "window": self.window_for_layer(index),
                "position": position,
            }, prefix + ".self_attn")
            feed_forward = PartSpec("gated_mlp", {
                "hidden_size": self.hidden_size,
                "intermediate_size": self.intermediate_size,
                "activation": self.hidden_act,
            }, prefix + ".mlp")
            layers.append(LayerSpec(
                block="pre_norm_residual",
                mixer=mixer,
                feed_forward=feed_forward,
                mixer_norm=norm.with_prefix(prefix + ".input_layernorm"),
                feed_forward_norm=norm.with_prefix(prefix + ".post_attention_layernorm"),
            ))
        spec = ModelSpec(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {
                "vocab_size": self.vocab_size, "hidden_size": self.hidden_size},
                "model.embed_tokens"),
            layers=tuple(layers),
            order=tuple(LayerCall(i) for i in range(self.num_hidden_layers)),
            final_norm=norm.with_prefix("model.norm"),
            head=PartSpec("lm_head", {
                "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "tied_to": "model.embed_tokens" if self.tie_word_embeddings else None},
                "lm_head"),
        )
        spec.validate()
        return spec


register_architecture(ARCHITECTURE, Qwen2Config)

"""Tiny configurations of the architecture for the tests.  They differ in every
size and option: layers, width, heads and groups, head size, feed-forward
width, vocabulary, rope base, eps, tied or own head, positions, window, page."""
import os

import torch

from tokenizer_b200 import Qwen2Config, write_random_model


def _cfg(**kw):
    base = dict(architectures=["Qwen2ForCausalLM"], hidden_act="silu")
    base.update(kw)
    return Qwen2Config.from_dict(base)


# name -> (config, seed, page size)
def tiny_a():
    return _cfg(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                intermediate_size=176, vocab_size=512, rope_theta=10000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=True, max_position_embeddings=128, use_sliding_window=False,
                sliding_window=64, max_window_layers=2), 0, 16


def tiny_b():
    return _cfg(num_hidden_layers=3, hidden_size=96, num_attention_heads=3, num_key_value_heads=1,
                intermediate_size=256, vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-5,
                tie_word_embeddings=False, max_position_embeddings=256, use_sliding_window=False,
                sliding_window=None, max_window_layers=3), 1, 8


def tiny_c():
    """The window on: layers 0-1 keep all keys, layers 2-3 the last 25 (two cache groups)."""
    return _cfg(num_hidden_layers=4, hidden_size=80, num_attention_heads=5, num_key_value_heads=5,
                head_dim=48, intermediate_size=112, vocab_size=301, rope_theta=500000.0,
                rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=512,
                use_sliding_window=True, sliding_window=24, max_window_layers=2), 2, 32


TINY = {"a": tiny_a, "b": tiny_b, "c": tiny_c}


def make_folder(tmp_path_factory, name, scale=None):
    config, seed, page = TINY[name]()
    folder = str(tmp_path_factory.mktemp(f"tiny_{name}"))
    write_random_model(folder, config, seed, scale=scale)
    return folder, config, page


def random_ids(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()

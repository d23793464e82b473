"""The plain implementation checked against hand-worked cases of the
reference's formulas (no GPU)."""
import math

import pytest
import torch

import plain_qwen2 as plain
from tiny import TINY, random_ids
from tokenizer_b200 import write_random_model


def test_mask_matrix_is_the_rule_entry_by_entry():
    for seq, window in ((1, None), (7, None), (9, 3), (12, 0), (6, 100)):
        rule = torch.tensor([[plain.mask_value(q, k, window) for k in range(seq)] for q in range(seq)])
        assert torch.equal(plain.attention_mask(seq, window), rule)


def test_logits_of_chosen_rows_are_rows_of_all_logits(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY["a"]()[0], 3)
    cfg, w = plain.load_folder(folder)
    ids = [3, 1, 4, 1, 5, 9, 2, 6]
    full = plain.all_logits(cfg, w, ids)
    assert torch.equal(plain.all_logits(cfg, w, ids, rows=[0, 5, 7]), full[[0, 5, 7]])


def test_mask_truth_table():
    # model.rs:1389-1399
    inf = -math.inf
    assert plain.mask_value(3, 3, None) == 0.0 and plain.mask_value(3, 4, None) == inf
    assert plain.mask_value(5, 0, None) == 0.0
    assert plain.mask_value(5, 2, 3) == 0.0 and plain.mask_value(5, 1, 3) == inf
    assert plain.mask_value(5, 6, 3) == inf


def test_rope_tables_and_rotation():
    cos, sin = plain.rope_tables(10000.0, 4, 3)
    assert cos.shape == (3, 2)
    assert torch.allclose(cos[0], torch.ones(2)) and torch.allclose(sin[0], torch.zeros(2))
    assert abs(float(sin[1, 0]) - math.sin(1.0)) < 1e-6
    assert abs(float(sin[2, 1]) - math.sin(2 * 10000.0 ** -0.5)) < 1e-6
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]])           # one head, one row at position 1
    out = plain.rope_apply(x, cos[1:2], sin[1:2])[0, 0]
    c0, s0, c1, s1 = float(cos[1, 0]), float(sin[1, 0]), float(cos[1, 1]), float(sin[1, 1])
    want = [1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 3 * c0 + 1 * s0, 4 * c1 + 2 * s1]
    assert torch.allclose(out, torch.tensor(want), atol=1e-6)
    # a rotation keeps the norm
    assert abs(float(out.norm()) - float(x.norm())) < 1e-5


def test_rms_norm_and_swiglu_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    y = plain.rms_norm(x, torch.tensor([1.0, 2.0]), 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[3 / r, 8 / r]]), atol=1e-6)
    w = {"p.gate_proj.weight": torch.tensor([[1.0, 0.0]]), "p.up_proj.weight": torch.tensor([[0.0, 2.0]]),
         "p.down_proj.weight": torch.tensor([[1.0], [-1.0]])}
    out = plain.swiglu_mlp(torch.tensor([[0.5, 3.0]]), w, "p.")
    silu = 0.5 / (1 + math.exp(-0.5))
    assert torch.allclose(out, torch.tensor([[silu * 6.0, -silu * 6.0]]), atol=1e-6)


def test_causality_and_the_window(tmp_path):
    config = TINY["c"]()[0]
    folder = write_random_model(str(tmp_path / "m"), config, 3, scale={r"(q|k)_proj\.weight": 8.0})
    cfg, w = plain.load_folder(folder)
    ids = random_ids(60, config.vocab_size, 1)
    full = plain.all_logits(cfg, w, ids)
    # a later token never changes an earlier row
    assert torch.equal(plain.all_logits(cfg, w, ids[:31])[:31], full[:31]) or \
        torch.allclose(plain.all_logits(cfg, w, ids[:31]), full[:31], atol=1e-6)
    # with the window off the far past matters; the config with it on differs
    cfg_off = dict(cfg, use_sliding_window=False)
    assert float((plain.all_logits(cfg_off, w, ids)[-1] - full[-1]).abs().max()) > 1e-4
    assert torch.allclose(plain.all_logits(cfg_off, w, ids)[:24], full[:24], atol=1e-6)


def test_greedy_ties_and_sampling_rules():
    assert plain.greedy_token(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1      # ties keep the lower id
    assert plain.greedy_token(torch.zeros(5)) == 0
    logits = torch.tensor([2.0, 1.0, 3.0, 0.0])
    assert plain.sample_token(logits, 0.0, 0.1, 0.99) == 2                    # temperature 0 is greedy
    kept, mass = plain.sample_intervals(logits, 1.0, 1.0)
    assert kept == [2, 0, 1, 3] and abs(mass[1] - math.exp(-1.0)) < 1e-6
    kept, _ = plain.sample_intervals(logits, 1.0, 0.7)                          # 0.644 < 0.7 <= 0.881
    assert kept == [2, 0]
    assert plain.sample_intervals(logits, 1.0, 0.0)[0] == [2]                 # at least one is kept
    probs = torch.softmax(logits, 0)
    assert plain.sample_token(logits, 1.0, 1.0, float(probs[2]) - 1e-3) == 2
    assert plain.sample_token(logits, 1.0, 1.0, float(probs[2]) + 1e-3) == 0
    assert plain.sample_token(logits, 1.0, 1.0, 0.9999) == 3
    # a low temperature sharpens
    assert plain.sample_intervals(logits, 0.1, 0.99)[0] == [2]

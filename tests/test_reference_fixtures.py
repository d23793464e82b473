"""Optional tests on the reference's own recorded outputs.  They need what cannot be committed
here: the real Qwen2.5-0.5B checkpoint and the reference's fixture files.  Set

    QWEN_INFER_MODEL     a folder with config.json, model.safetensors (and tokenizer.json)
    QWEN_INFER_FIXTURES  the reference's tests/fixtures folder (qwen_last_logits.f32,
                         qwen_greedy.json, qwen_cases.jsonl)

and they compare, as the reference's own test does (qwen-infer/tests/reference.rs:15-65): the
float32 logits at the last position of the fixture's prompt ids with the recorded ones (max
|diff| <= 1e-3) and the 20 greedy ids, for the plain implementation under tests/ and for the
engine in 32-bit; in bfloat16 the engine's best id and most of its 16 best; and the byte-level
BPE with the recorded (text, ids) pairs.  Without the two variables every test here is skipped,
and the plain implementation rests on the reference's formulas alone."""
import json
import os

import numpy as np
import pytest
import torch

import plain_qwen2 as plain

MODEL = os.environ.get("QWEN_INFER_MODEL")
FIXTURES = os.environ.get("QWEN_INFER_FIXTURES")


def _have(*names):
    return bool(MODEL and FIXTURES and os.path.exists(os.path.join(MODEL, "model.safetensors"))
                and all(os.path.exists(os.path.join(FIXTURES, n)) for n in names))


needs_model = pytest.mark.skipif(
    not _have("qwen_last_logits.f32", "qwen_greedy.json"),
    reason="set QWEN_INFER_MODEL (the real checkpoint) and QWEN_INFER_FIXTURES (the reference's fixtures)")


def recorded():
    with open(os.path.join(FIXTURES, "qwen_greedy.json")) as fh:
        meta = json.load(fh)
    logits = np.fromfile(os.path.join(FIXTURES, "qwen_last_logits.f32"), dtype="<f4")
    assert logits.size == meta["vocab"]
    return meta, torch.from_numpy(logits.copy())


@needs_model
def test_the_plain_implementation_gives_the_recorded_logits_and_greedy_ids():
    meta, want = recorded()
    cfg, w = plain.load_folder(MODEL)
    got = plain.all_logits(cfg, w, meta["prompt_ids"])[-1]
    assert got.shape == want.shape
    assert float((got - want).abs().max()) <= 1e-3
    assert plain.greedy_generate(cfg, w, meta["prompt_ids"], len(meta["greedy_ids"])) == meta["greedy_ids"]


@needs_model
@pytest.mark.gpu
def test_the_engine_in_32_bit_gives_the_recorded_logits_and_greedy_ids():
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    meta, want = recorded()
    model = tb.load_model(MODEL, dtype="float32")
    engine = tb.engine_for(model, 64, 16, max_requests=1)
    cache = engine.cache.open("fixture")
    ids = meta["prompt_ids"]
    engine.cache.reserve(cache, len(ids))
    got = engine.step([StepEntry(cache, ids, [len(ids) - 1])]).cpu()[0]
    assert float((got - want).abs().max()) <= 1e-3
    assert tb.greedy_tokens(model, ids, len(meta["greedy_ids"])) == meta["greedy_ids"]


@needs_model
@pytest.mark.gpu
def test_the_engine_in_bfloat16_agrees_on_the_best_ids():
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    meta, want = recorded()
    model = tb.load_model(MODEL, dtype="bfloat16")
    engine = tb.engine_for(model, 64, 16, max_requests=1)
    cache = engine.cache.open("fixture")
    ids = meta["prompt_ids"]
    engine.cache.reserve(cache, len(ids))
    got = engine.step([StepEntry(cache, ids, [len(ids) - 1])]).float().cpu()[0]
    assert int(got.argmax()) == meta["argmax"]
    best = set(torch.topk(want, 16).indices.tolist())
    assert len(best & set(torch.topk(got, 16).indices.tolist())) >= 12
    assert float((got - want).abs().max()) <= 2e-2 * float(want.abs().max())


@pytest.mark.skipif(not (_have("qwen_cases.jsonl") and os.path.exists(os.path.join(MODEL or "", "tokenizer.json"))),
                    reason="needs the real tokenizer.json and the reference's qwen_cases.jsonl")
def test_the_byte_level_bpe_gives_the_recorded_ids():
    from tokenizer_b200.text import ByteLevelBPE
    tokenizer = ByteLevelBPE.from_file(os.path.join(MODEL, "tokenizer.json"))
    with open(os.path.join(FIXTURES, "qwen_cases.jsonl")) as fh:
        cases = [json.loads(line) for line in fh if line.strip()]
    assert cases
    for case in cases:
        assert tokenizer.encode(case["text"]) == case["ids"], case["text"]
        assert tokenizer.decode(case["ids"]) == case["text"]

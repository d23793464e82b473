"""Stop conditions, streaming text and the draws of a request (no GPU).  The
cases follow the reference's generate.rs:503-749, stream.rs:80-142 and
lib.rs:135-149, with a scripted byte codec in place of a tokenizer."""
import json

import pytest

from fake_engine import FakeEngine
from tokenizer_b200.api import generate, generate_with, load_eos_token_ids
from tokenizer_b200.engine.generate import (Control, GenerateParams, SampleCursor, StopHold,
                                            StopReason, StreamDecoder)
from tokenizer_b200.sampling import uniform, validate_sampling


def feed(cursor, ids):
    for token in ids:
        if not cursor.wants_sample():
            break
        if not cursor.accept(token):
            break
    return cursor.done


def codec(table):
    return lambda token: table[token]


def test_max_tokens_and_eos():
    c = SampleCursor(GenerateParams(max_tokens=3))
    out = feed(c, [5, 6, 7, 8])
    assert out.tokens == [5, 6, 7] and out.reason == StopReason.MAX_TOKENS and out.completion_tokens == 3
    c = SampleCursor(GenerateParams(max_tokens=5, eos=[9, 11]))
    out = feed(c, [5, 11, 7])
    assert out.tokens == [5] and out.reason == StopReason.EOS
    assert out.completion_tokens == 2            # the EOS id counts but is not kept
    c = SampleCursor(GenerateParams(max_tokens=0))
    assert not c.wants_sample() and c.done.reason == StopReason.MAX_TOKENS and c.done.tokens == []


def test_stop_string_across_tokens_is_held_back():
    table = {1: b"Hello", 2: b" wor", 3: b"ld", 4: b"!"}
    seen = []
    c = SampleCursor(GenerateParams(max_tokens=9, stop=["world"]), codec(table),
                     lambda piece: seen.append(piece) or Control.CONTINUE)
    out = feed(c, [1, 2, 3, 4])
    assert out.reason == StopReason.STOP_STRING
    assert out.text == "Hello " and out.tokens == [1, 2, 3]      # the completing id is kept
    assert "".join(seen) == "Hello " and all("wor" not in s for s in seen)
    # a prefix that turns out to be ordinary text is released
    table = {1: b"a wo", 2: b"nder"}
    c = SampleCursor(GenerateParams(max_tokens=2, stop=["world"]), codec(table))
    assert feed(c, [1, 2]).text == "a wonder"


def test_cancel_keeps_the_token_and_runs_no_more():
    table = {1: b"a", 2: b"b", 3: b"c"}
    c = SampleCursor(GenerateParams(max_tokens=9), codec(table),
                     lambda piece: Control.STOP if piece == "b" else Control.CONTINUE)
    out = feed(c, [1, 2, 3])
    assert out.reason == StopReason.CANCELLED and out.tokens == [1, 2] and out.text == "ab"


def test_split_utf8_waits_and_illegal_bytes_are_replaced():
    d = StreamDecoder()
    euro = "€".encode()
    assert d.push(euro[:1]) == "" and d.push(euro[1:2]) == "" and d.push(euro[2:]) == "€"
    assert d.push(b"\xff") == "�"
    assert d.push(b"ok\xe2") == "ok" and d.finish() == "�"
    table = {1: euro[:2], 2: euro[2:] + b"x"}
    c = SampleCursor(GenerateParams(max_tokens=2), codec(table))
    out = feed(c, [1, 2])
    assert out.text == "€x" and out.chunks == ["€x"]
    c = SampleCursor(GenerateParams(max_tokens=1), codec(table))
    assert feed(c, [1]).text == "�"          # flushed at the end only


def test_stop_hold():
    h = StopHold()
    assert h.push("ab", ["bcd"]) == (False, "a")
    assert h.push("c", ["bcd"]) == (False, "")
    assert h.push("x", ["bcd"]) == (False, "bcx")
    assert h.push("bcd!", ["bcd"]) == (True, "")


def test_params_are_validated():
    for bad in (dict(temperature=float("nan")), dict(temperature=-0.5), dict(top_p=-0.1),
                dict(top_p=float("inf")), dict(stop=[""]), dict(max_tokens=-1)):
        with pytest.raises(ValueError):
            SampleCursor(GenerateParams(**bad))
    with pytest.raises(ValueError, match="tokenizer"):
        SampleCursor(GenerateParams(stop=["x"]))
    validate_sampling(0.0, 0.0)


def test_draws_are_a_function_of_seed_and_count():
    a = [uniform(3, k) for k in range(1000)]
    assert a == [uniform(3, k) for k in range(1000)]
    assert all(0.0 <= u < 1.0 for u in a) and len(set(a)) > 990
    assert abs(sum(a) / 1000 - 0.5) < 0.05
    assert a[:5] != [uniform(4, k) for k in range(5)]
    c = SampleCursor(GenerateParams(max_tokens=5, temperature=1.0, seed=3))
    assert c.next_uniform() == a[0]
    c.accept(1)
    assert c.next_uniform() == a[1]


def test_eos_ids_from_generation_config(tmp_path):
    p = tmp_path / "generation_config.json"
    p.write_text(json.dumps({"eos_token_id": [151645, 151643]}))
    assert load_eos_token_ids(str(p)) == [151645, 151643]
    assert load_eos_token_ids(str(tmp_path)) == [151645, 151643]
    p.write_text(json.dumps({"eos_token_id": 7}))
    assert load_eos_token_ids(str(p)) == [7]
    p.write_text(json.dumps({"eos_token_id": "x"}))
    with pytest.raises(ValueError):
        load_eos_token_ids(str(p))
    assert load_eos_token_ids(str(tmp_path / "none")) == []


def test_entry_point_on_the_fake_engine():
    engine = FakeEngine(num_pages=64, max_requests=1)
    out = generate(engine, [1, 2, 3], GenerateParams(max_tokens=4))
    assert len(out.tokens) == 4 and out.reason == StopReason.MAX_TOKENS
    pieces = []
    table = {t: bytes([65 + t % 26]) for t in range(50)}
    out2 = generate_with(FakeEngine(num_pages=64, max_requests=1), [1, 2, 3], GenerateParams(max_tokens=4),
                         lambda t: table[t], lambda s: pieces.append(s) or Control.CONTINUE)
    assert out2.tokens == out.tokens and "".join(pieces) == out2.text and len(out2.text) == 4

"""The byte-level BPE and the command line's argument handling (no GPU), on a
synthetic tokenizer.json: the 256 byte tokens, a few merges, two added tokens
(the shape of the reference's own synthetic file, src/qwen.rs:376-453)."""
import json

import pytest

from tokenizer_b200.cli import UsageError, parse_args
from tokenizer_b200.text import ByteLevelBPE, TokenizerError
from tokenizer_b200.text.bpe import _byte_alphabet

QWEN_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*"
                r"|\s*[\r\n]+|\s+(?!\S)|\s+")


def synthetic(merges=("h e", "l l", "he ll", "Ġ w", "hell o"), added=("<|end|>", "<|endoftext|>")):
    inverse = {b: c for c, b in _byte_alphabet().items()}
    vocab = {inverse[b]: b for b in range(256)}
    for merge in merges:
        left, right = merge.split(" ")
        vocab[left + right] = len(vocab)
    return {
        "normalizer": {"type": "NFC"},
        "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
            {"type": "Split", "pattern": {"Regex": QWEN_PATTERN}, "behavior": "Isolated", "invert": False},
            {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": False, "use_regex": False}]},
        "model": {"type": "BPE", "vocab": vocab, "merges": list(merges)},
        "added_tokens": [{"id": len(vocab) + i, "content": a, "normalized": False}
                         for i, a in enumerate(added)],
    }


def test_alphabet():
    table = _byte_alphabet()
    assert len(table) == 256 and sorted(table.values()) == list(range(256))
    assert table["A"] == 65 and table["Ġ"] == 32 and table["Ċ"] == 10 and table["ÿ"] == 255


def test_merges_by_rank_and_round_trip():
    bpe = ByteLevelBPE.from_dict(synthetic())
    hello = 256 + 4
    assert bpe.encode("hello") == [hello]
    assert bpe.encode("hello world") == [hello, 256 + 3, ord("o"), ord("r"), ord("l"), ord("d")]
    # "ll" outranks "hell" only through its parts: h e | l l -> he ll -> hell o
    assert bpe.encode("hell") == [256 + 2]
    assert bpe.encode("shell") == [ord("s"), 256 + 2]
    for text in ["hello world", "naïve café ☕ 12 34", "a\n\n b\t", "  spaces  ", "€", "it's"]:
        assert bpe.decode(bpe.encode(text)) == text
    assert bpe.encode("") == []


def test_added_tokens_are_cut_first_and_longest_wins():
    raw = synthetic()
    bpe = ByteLevelBPE.from_dict(raw)
    end = raw["added_tokens"][0]["id"]
    assert bpe.encode("hello<|end|>hello") == [260, end, 260]
    assert bpe.encode("<|endoftext|>") == [end + 1]
    assert bpe.decode_bytes([end]) == b"<|end|>"
    with pytest.raises(TokenizerError, match="unknown token id"):
        bpe.decode_bytes([99999])


def test_nfc_and_digits():
    bpe = ByteLevelBPE.from_dict(synthetic())
    assert bpe.encode("é") == bpe.encode("é")          # composed before encoding
    assert bpe.encode("12") == [ord("1"), ord("2")]               # \p{N} one at a time


@pytest.mark.parametrize("change, message", [
    (lambda r: r.pop("normalizer"), "no normalizer"),
    (lambda r: r["normalizer"].update(type="NFKC"), "NFC"),
    (lambda r: r["pre_tokenizer"].update(type="ByteLevel"), "Sequence"),
    (lambda r: r["pre_tokenizer"]["pretokenizers"][0].update(behavior="Removed"), "Isolated"),
    (lambda r: r["pre_tokenizer"]["pretokenizers"][0].update(invert=True), "invert"),
    (lambda r: r["pre_tokenizer"]["pretokenizers"][1].update(use_regex=True), "use_regex"),
    (lambda r: r["model"].update(type="WordPiece"), "BPE"),
    (lambda r: r["model"]["vocab"].pop("A"), "missing single-byte token 65"),
    (lambda r: r["model"]["merges"].append("q q"), "concatenation"),
    (lambda r: r["model"]["merges"].append("hello"), "two bytes_to_unicode"),
    (lambda r: r["added_tokens"][0].update(normalized=True), "normalized"),
    (lambda r: r["added_tokens"][0].update(id=65), "already belongs"),
    (lambda r: r["model"]["vocab"].update({"中": 999}), "bytes_to_unicode scalar"),
])
def test_the_file_must_say_what_the_reader_does(change, message):
    raw = json.loads(json.dumps(synthetic()))
    change(raw)
    with pytest.raises(TokenizerError, match=message):
        ByteLevelBPE.from_dict(raw)


def test_command_line_options():
    args = parse_args(["--max-tokens", "5", "--temperature", "0.7", "--top-p", "0.9", "--seed", "3",
                       "--stop", "a", "--stop", "b", "The capital"])
    assert (args["max_tokens"], args["temperature"], args["top_p"], args["seed"]) == (5, 0.7, 0.9, 3)
    assert args["stop"] == ["a", "b"] and args["prompt"] == "The capital"
    d = parse_args(["x"])
    assert (d["max_tokens"], d["temperature"], d["top_p"], d["seed"], d["stop"]) == (20, 0.0, 1.0, 0, [])
    assert parse_args(["--ids", "1,2,3"])["ids"] == [1, 2, 3]
    for bad in (["--nope"], ["a", "b"], ["--max-tokens"], ["--max-tokens", "x", "p"]):
        with pytest.raises(UsageError):
            parse_args(bad)

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
    (lambda r: r["pre_tokenizer"]["pretokenizers"][0].update(invert=True), "inverted"),
    (lambda r: r["pre_tokenizer"]["pretokenizers"][1].update(use_regex=True), "use_regex"),
    (lambda r: r["model"].update(type="WordPiece"), "BPE"),
    (lambda r: r["model"]["vocab"].pop("A"), "no token for the single byte 65"),
    (lambda r: r["model"]["merges"].append("q q"), "produces bytes the vocab does not hold"),
    (lambda r: r["model"]["merges"].append("hello"), "not a pair of tokens"),
    (lambda r: r["added_tokens"][0].update(normalized=True), "normalization"),
    (lambda r: r["added_tokens"][0].update(id=65), "taken by a vocab token"),
    (lambda r: r["model"]["vocab"].update({"中": 999}), "stands for no byte"),
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
    assert args["stop"] == ["a", "b"] and args["prompts"] == ["The capital"]
    d = parse_args(["x"])
    assert (d["max_tokens"], d["temperature"], d["top_p"], d["seed"], d["stop"]) == (20, 0.0, 1.0, 0, [])
    assert parse_args(["--ids", "1,2,3"])["ids"] == [[1, 2, 3]]
    assert (d["num_pages"], d["page_size"], d["max_batch_size"], d["token_budget"]) == (None, 16, 8, 2048)
    # several prompts, and the sizes of the cache and of the scheduler (under either name)
    many = parse_args(["--ids", "1,2", "--ids", "3", "--num-pages", "7", "--page-size", "8",
                       "--max-batch-size", "2", "--token-budget", "24"])
    assert many["ids"] == [[1, 2], [3]]
    assert (many["num_pages"], many["page_size"], many["max_batch_size"], many["token_budget"]) == (7, 8, 2, 24)
    alias = parse_args(["--num-blocks", "9", "--block-size", "4", "--prefill-chunk", "5", "a", "b"])
    assert (alias["num_pages"], alias["page_size"], alias["token_budget"]) == (9, 4, 5)
    assert alias["prompts"] == ["a", "b"]
    for bad in (["--nope"], ["a", "--ids", "1"], ["--max-tokens"], ["--max-tokens", "x", "p"],
                ["--num-pages", "0", "p"], ["--page-size", "x", "p"]):
        with pytest.raises(UsageError):
            parse_args(bad)

"""Text to ids and back for the command line: the byte-level BPE of a Qwen
`tokenizer.json` (reference: src/qwen.rs:137-297 for the file, src/rank.rs:
333-447, 485-649 for encoding).  The file must say what this reader does: NFC
normalisation, a Split step (Isolated, not inverted) whose regular expression is
taken from the file, a ByteLevel step without its own regex, a BPE model.

Vocabulary strings are written in the GPT-2 "bytes to unicode" alphabet and are
mapped back to raw bytes; a merge's rank is its index in the merges list; added
tokens (all `normalized: false`) are cut out of the text before anything else,
leftmost first and the longer one on a tie.  A piece is encoded by starting from
its bytes and merging, again and again, the adjacent pair whose concatenation
has the lowest rank (the leftmost on a tie)."""
from __future__ import annotations

import json
import unicodedata
from typing import Dict, List, Tuple


class TokenizerError(ValueError):
    pass


def _byte_alphabet() -> Dict[str, int]:
    """Character -> byte of the bytes-to-unicode alphabet: printable bytes stand
    for themselves, the other 68 take U+0100 upward in byte order."""
    own = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, extra = {}, 0
    for byte in range(256):
        if byte in own:
            table[chr(byte)] = byte
        else:
            table[chr(256 + extra)] = byte
            extra += 1
    return table


class ByteLevelBPE:
    def __init__(self, vocab: Dict[bytes, int], ranks: Dict[bytes, int], added: Dict[str, int],
                 pattern: str):
        import regex
        self.vocab = vocab
        self.ranks = ranks
        self.added = added
        self.pattern = regex.compile(pattern)
        size = max(list(vocab.values()) + list(added.values())) + 1
        self.id_to_bytes: List[bytes] = [None] * size
        for data, token in vocab.items():
            self.id_to_bytes[token] = data
        for text, token in added.items():
            self.id_to_bytes[token] = text.encode()
        # added tokens by first character, longest first, for the leftmost scan
        self._added_sorted = sorted(added, key=len, reverse=True)

    # ---- loading ------------------------------------------------------------------
    @classmethod
    def from_file(cls, path: str) -> "ByteLevelBPE":
        try:
            with open(path, encoding="utf-8") as fh:
                raw = json.load(fh)
        except OSError as err:
            raise TokenizerError(f"cannot read {path}: {err}") from None
        except json.JSONDecodeError as err:
            raise TokenizerError(f"{path} is not JSON: {err}") from None
        return cls.from_dict(raw)

    @classmethod
    def from_dict(cls, raw: dict) -> "ByteLevelBPE":
        normalizer = raw.get("normalizer")
        if not normalizer:
            raise TokenizerError("the file names no normalizer (this tokenizer normalizes to NFC)")
        if normalizer.get("type") != "NFC":
            raise TokenizerError(f"the normalizer is {normalizer.get('type')}; only NFC is handled")
        pre = raw.get("pre_tokenizer") or {}
        if pre.get("type") != "Sequence":
            raise TokenizerError(f"the pre-tokenizer is {pre.get('type')}; a Sequence of Split and ByteLevel is handled")
        steps = pre.get("pretokenizers", [])
        split = next((s for s in steps if s.get("type") == "Split"), None)
        if split is None:
            raise TokenizerError("the pre-tokenizer Sequence lacks its Split step")
        if split.get("behavior") != "Isolated":
            raise TokenizerError(f"the Split step behaves as {split.get('behavior')}; only Isolated is handled")
        if split.get("invert", False):
            raise TokenizerError("the Split step is inverted (invert: true), which is not handled")
        pattern = (split.get("pattern") or {}).get("Regex")
        if not pattern:
            raise TokenizerError("the Split step gives no Regex pattern")
        byte_level = next((s for s in steps if s.get("type") == "ByteLevel"), None)
        if byte_level is None:
            raise TokenizerError("the pre-tokenizer Sequence lacks its ByteLevel step")
        if byte_level.get("use_regex", False):
            raise TokenizerError("the ByteLevel step has use_regex on; splitting belongs to the Split step alone")
        model = raw.get("model") or {}
        if model.get("type") != "BPE":
            raise TokenizerError(f"the model is {model.get('type')}; only BPE is handled")

        alphabet = _byte_alphabet()

        def to_bytes(token: str) -> bytes:
            try:
                return bytes(alphabet[ch] for ch in token)
            except KeyError as err:
                raise TokenizerError(
                    f"a vocab entry holds U+{ord(err.args[0]):04X}, which stands for no byte in the byte-level alphabet") from None

        vocab: Dict[bytes, int] = {}
        ids = set()
        for token, token_id in model.get("vocab", {}).items():
            data = to_bytes(token)
            if data in vocab:
                raise TokenizerError(f"id {token_id} spells bytes that another id already spells")
            if token_id in ids:
                raise TokenizerError(f"id {token_id} is given to two vocab entries")
            vocab[data] = token_id
            ids.add(token_id)
        for byte in range(256):
            if bytes([byte]) not in vocab:
                raise TokenizerError(f"the vocab has no token for the single byte {byte}")
        ranks: Dict[bytes, int] = {}
        for index, merge in enumerate(model.get("merges", [])):
            parts = merge.split(" ") if isinstance(merge, str) else list(merge)
            if len(parts) != 2 or not parts[0] or not parts[1]:
                raise TokenizerError(f"merge {index} is not a pair of tokens in the byte-level alphabet")
            left, right = to_bytes(parts[0]), to_bytes(parts[1])
            if left not in vocab or right not in vocab:
                raise TokenizerError(f"merge {index} joins a token the vocab does not hold")
            if left + right not in vocab:
                raise TokenizerError(f"merge {index} produces bytes the vocab does not hold")
            if left + right in ranks:
                raise TokenizerError(f"merge {index} produces bytes an earlier merge already produces")
            ranks[left + right] = index
        added: Dict[str, int] = {}
        for entry in raw.get("added_tokens", []):
            if entry.get("normalized", True):
                raise TokenizerError(
                    f"added token {entry.get('content')!r} asks for normalization; added tokens are matched as written")
            if not entry.get("content"):
                raise TokenizerError("an added token has no content")
            if entry["id"] in ids:
                raise TokenizerError(f"added token id {entry['id']} is taken by a vocab token")
            if entry["content"] in added:
                raise TokenizerError(f"added token {entry['content']!r} appears twice")
            added[entry["content"]] = entry["id"]
        return cls(vocab, ranks, added, pattern)

    # ---- encoding ------------------------------------------------------------------
    def _cut_added(self, text: str) -> List[Tuple[bool, str]]:
        """[(is an added token, piece)]: leftmost match first, the longer on a tie."""
        if not self.added:
            return [(False, text)]
        out, start, at = [], 0, 0
        while at < len(text):
            hit = next((a for a in self._added_sorted if text.startswith(a, at)), None)
            if hit is None:
                at += 1
                continue
            if at > start:
                out.append((False, text[start:at]))
            out.append((True, hit))
            at += len(hit)
            start = at
        if start < len(text):
            out.append((False, text[start:]))
        return out

    def _merge(self, piece: bytes) -> List[int]:
        parts = [piece[i:i + 1] for i in range(len(piece))]
        while len(parts) > 1:
            best_rank, best_at = None, -1
            for i in range(len(parts) - 1):
                rank = self.ranks.get(parts[i] + parts[i + 1])
                if rank is not None and (best_rank is None or rank < best_rank):
                    best_rank, best_at = rank, i
            if best_rank is None:
                break
            parts[best_at:best_at + 2] = [parts[best_at] + parts[best_at + 1]]
        return [self.vocab[p] for p in parts]

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        for is_added, segment in self._cut_added(text):
            if is_added:
                ids.append(self.added[segment])
                continue
            segment = unicodedata.normalize("NFC", segment)
            at = 0
            for match in self.pattern.finditer(segment):
                if match.start() > at:                       # a gap the pattern skipped is a piece too
                    ids += self._merge(segment[at:match.start()].encode())
                if match.end() > match.start():
                    ids += self._merge(match.group().encode())
                at = match.end()
            if at < len(segment):
                ids += self._merge(segment[at:].encode())
        return ids

    # ---- decoding ------------------------------------------------------------------
    def decode_bytes(self, ids) -> bytes:
        out = bytearray()
        for token in ids:
            if not 0 <= token < len(self.id_to_bytes) or self.id_to_bytes[token] is None:
                raise TokenizerError(f"unknown token id {token}")
            out += self.id_to_bytes[token]
        return bytes(out)

    def decode(self, ids) -> str:
        return self.decode_bytes(ids).decode("utf-8")

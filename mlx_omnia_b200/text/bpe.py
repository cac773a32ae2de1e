"""Byte-level BPE read from a checkpoint's `tokenizer.json`.

What the file declares is what is done: the pre-tokenizer's stages (regex splits and the
byte-level stage), the vocabulary, the ranked merges, whether a pre-token that is already in
the vocabulary skips the merges (`ignore_merges`), and the added tokens, which are cut out of
the text before anything else sees it. A stage this reader does not know raises instead of
tokenizing differently from the checkpoint. The reference reads the same file with the same
meaning (src/mlx_omnia/engine/bpe.py:115-295) and wires it into the model facade
(src/mlx_omnia/engine/models/muse_glimmer/checkpoint.py:113-119).

Merging works on vocabulary ids, not strings: a pre-token becomes the ids of its bytes, and
`merges[(left id, right id)] = (rank, merged id)` is looked up for neighbours; the pair of
lowest rank is joined (every occurrence, left to right) until no neighbouring pair has a rank.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import regex

# The pattern a ByteLevel stage splits with when it says `use_regex` (the GPT-2 one).
_BYTE_LEVEL_PATTERN = r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"


def _byte_alphabet() -> list[str]:
    """One printable character per byte value: the printable Latin-1 ranges stand for themselves,
    every other byte gets the next code point from 256 on (the byte-level alphabet of GPT-2)."""
    keep = [*range(0x21, 0x7F), *range(0xA1, 0xAD), *range(0xAE, 0x100)]
    table, spare = [""] * 256, 256
    for value in range(256):
        if value in keep:
            table[value] = chr(value)
        else:
            table[value] = chr(spare)
            spare += 1
    return table


BYTE_TO_CHAR = _byte_alphabet()
CHAR_TO_BYTE = {char: value for value, char in enumerate(BYTE_TO_CHAR)}


@dataclass(frozen=True)
class _Stage:
    """One split of the pre-tokenizer: where `pattern` matches, the text is cut; `keep` says what
    happens to the match itself ("alone": a piece of its own, "next": glued to the piece after
    it, "previous": glued to the piece before it, "drop": removed)."""

    pattern: "regex.Pattern[str]"
    keep: str

    def cut(self, text: str) -> list[str]:
        pieces: list[str] = []
        at = 0  # start of the piece being gathered
        for match in self.pattern.finditer(text):
            lo, hi = match.span()
            if lo == hi:
                continue
            if self.keep == "alone":
                pieces += [text[at:lo], text[lo:hi]]
                at = hi
            elif self.keep == "next":
                pieces.append(text[at:lo])
                at = lo
            elif self.keep == "previous":
                pieces.append(text[at:hi])
                at = hi
            else:  # drop
                pieces.append(text[at:lo])
                at = hi
        pieces.append(text[at:])
        return [piece for piece in pieces if piece]


_BEHAVIOURS = {"Isolated": "alone", "MergedWithNext": "next", "MergedWithPrevious": "previous", "Removed": "drop"}


def _stages(declared: dict | None) -> tuple[list[_Stage], bool]:
    """The pre-tokenizer as a list of splits, and whether a space is put before the text."""
    if declared is None:
        return [], False
    steps = declared.get("pretokenizers", []) if declared.get("type") == "Sequence" else [declared]
    stages, prefix_space = [], False
    for step in steps:
        kind = step.get("type")
        if kind == "Split":
            pattern = step.get("pattern", {})
            source = pattern.get("Regex") if "Regex" in pattern else regex.escape(pattern.get("String", ""))
            behaviour = step.get("behavior", "Isolated")
            if not source or behaviour not in _BEHAVIOURS:
                raise ValueError(f"tokenizer.json: a Split stage this reader does not know: {step}")
            if step.get("invert", False):
                raise ValueError("tokenizer.json: inverted Split stages are not read")
            stages.append(_Stage(regex.compile(source), _BEHAVIOURS[behaviour]))
        elif kind == "ByteLevel":
            prefix_space = prefix_space or bool(step.get("add_prefix_space", False))
            if step.get("use_regex", False):
                stages.append(_Stage(regex.compile(_BYTE_LEVEL_PATTERN), "alone"))
        else:
            raise ValueError(f"tokenizer.json: pre-tokenizer stage {kind!r} is not read")
    return stages, prefix_space


class ByteLevelBPE:
    def __init__(self, vocab: dict[str, int], merges: list, added: dict[str, int], stages: list[_Stage],
                 prefix_space: bool = False, ignore_merges: bool = False) -> None:
        self.vocab, self.added, self.stages = vocab, added, stages
        self.prefix_space, self.ignore_merges = prefix_space, ignore_merges
        self.byte_ids = [vocab.get(char, -1) for char in BYTE_TO_CHAR]
        self.merges: dict[tuple[int, int], tuple[int, int]] = {}
        for rank, merge in enumerate(merges):
            left, right = merge.split(" ", 1) if isinstance(merge, str) else merge
            if left in vocab and right in vocab and left + right in vocab:
                self.merges[(vocab[left], vocab[right])] = (rank, vocab[left + right])
        # What an id turns back into: the bytes of its symbol, or an added token's own text.
        self.pieces: dict[int, bytes] = {}
        for symbol, index in vocab.items():
            if symbol in added:
                continue
            try:
                self.pieces[index] = bytes(CHAR_TO_BYTE[char] for char in symbol)
            except KeyError:
                raise ValueError(f"tokenizer.json: {symbol!r} is neither byte-level nor an added token") from None
        for content, index in added.items():
            self.pieces[index] = content.encode("utf-8")
        # Added tokens are looked for first, the longest first where one starts another.
        self._added = regex.compile("|".join(regex.escape(t) for t in sorted(added, key=len, reverse=True))) \
            if added else None

    @classmethod
    def from_file(cls, path: str | Path) -> "ByteLevelBPE":
        raw = json.loads(Path(path).read_text(encoding="utf-8"))
        model = raw.get("model", {})
        if model.get("type", "BPE") != "BPE":
            raise ValueError(f"tokenizer.json: a {model.get('type')} model is not a byte-level BPE")
        stages, prefix_space = _stages(raw.get("pre_tokenizer"))
        added = {entry["content"]: int(entry["id"]) for entry in raw.get("added_tokens", [])}
        return cls(dict(model["vocab"]), list(model.get("merges", [])), added, stages, prefix_space,
                   bool(model.get("ignore_merges", False)))

    @property
    def vocab_size(self) -> int:
        return max(self.pieces, default=-1) + 1

    # -- text -> ids -------------------------------------------------------------------------------
    def _merge(self, ids: list[int]) -> list[int]:
        while len(ids) > 1:
            best = None  # (rank, merged id, left id, right id) of the neighbouring pair of lowest rank
            for pair in zip(ids, ids[1:]):
                found = self.merges.get(pair)
                if found is not None and (best is None or found[0] < best[0]):
                    best = (found[0], found[1], pair[0], pair[1])
            if best is None:
                break
            _, merged, left, right = best
            out, i = [], 0
            while i < len(ids):
                if i + 1 < len(ids) and ids[i] == left and ids[i + 1] == right:
                    out.append(merged)
                    i += 2
                else:
                    out.append(ids[i])
                    i += 1
            ids = out
        return ids

    def _plain(self, text: str) -> list[int]:
        """Ids of text that holds no added token."""
        if self.prefix_space and text and not text.startswith(" "):
            text = " " + text
        pieces = [text]
        for stage in self.stages:
            pieces = [part for piece in pieces for part in stage.cut(piece)]
        ids: list[int] = []
        for piece in pieces:
            data = piece.encode("utf-8")
            if self.ignore_merges:
                whole = self.vocab.get("".join(BYTE_TO_CHAR[b] for b in data))
                if whole is not None:
                    ids.append(whole)
                    continue
            start = [self.byte_ids[b] for b in data]
            if -1 in start:
                raise ValueError("tokenizer.json: the vocabulary lacks a single byte; the text cannot be encoded")
            ids += self._merge(start)
        return ids

    def encode(self, text: str) -> list[int]:
        if self._added is None:
            return self._plain(text)
        ids, at = [], 0
        for match in self._added.finditer(text):
            ids += self._plain(text[at: match.start()])
            ids.append(self.added[match.group()])
            at = match.end()
        return ids + self._plain(text[at:])

    # -- ids -> text -------------------------------------------------------------------------------
    def decode_bytes(self, ids) -> bytes:
        try:
            return b"".join(self.pieces[int(i)] for i in ids)
        except KeyError as missing:
            raise ValueError(f"token id {missing.args[0]} is not in the tokenizer's vocabulary") from None

    def decode(self, ids) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")


class Detokenizer:
    """Turns ids into text one at a time without ever cutting a character in two: bytes that do
    not yet end a UTF-8 character wait for the ids that complete them."""

    def __init__(self, tokenizer) -> None:
        self.tokenizer = tokenizer
        self.held = b""

    def feed(self, token_id: int) -> str:
        decode_bytes = getattr(self.tokenizer, "decode_bytes", None)
        if decode_bytes is None:  # a tokenizer without bytes (ids as decimal text): nothing can be cut
            return self.tokenizer.decode([token_id])
        data = self.held + decode_bytes([token_id])
        cut = len(data)
        for back in range(1, min(3, len(data)) + 1):
            byte = data[-back]
            if byte >= 0xC0:  # the first byte of a character of 2, 3 or 4 bytes
                if back < (2 if byte < 0xE0 else 3 if byte < 0xF0 else 4):
                    cut = len(data) - back  # it has not all its bytes yet
                break
            if byte < 0x80:
                break  # ASCII: whatever precedes is complete
        self.held = data[cut:]
        return data[:cut].decode("utf-8", errors="replace")

    def flush(self) -> str:
        text, self.held = self.held.decode("utf-8", errors="replace"), b""
        return text

"""GPT-2's byte-level BPE tokenizer, read from the ``vocab.json`` and ``merges.txt`` of a model
folder (the reference's crates/core/src/tokenizer.rs, whose steps these are).

  1. Pre-tokenise: split the text into chunks by a fixed rule: contractions ('s 't 're 've 'm 'll
     'd), runs of letters, runs of digits, runs of other symbols (each optionally led by ONE space),
     and whitespace, where a run of whitespace that is followed by something else leaves its last
     character behind as the next chunk's leading space (tokenizer.rs:150-227).  Merges never cross
     a chunk's boundary.
  2. Bytes to symbols: a chunk is its UTF-8 bytes; each of the 256 bytes has a token of its own, so
     any text can be encoded.
  3. Merge: the adjacent pair with the lowest rank in ``merges.txt`` is merged, again and again,
     until none is left (tokenizer.rs:123-141).
Decoding concatenates the tokens' bytes and reads them as UTF-8 (invalid bytes become U+FFFD).

``vocab.json`` and ``merges.txt`` are text files but tokens are byte strings: the files write each
byte as a printable character (the printable bytes 0x21-0x7E, 0xA1-0xAC and 0xAE-0xFF as themselves,
the others as U+0100 and up in byte order; tokenizer.rs:35-49), which is undone at load.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Tuple

END_OF_TEXT = "<|endoftext|>"


def bytes_to_unicode() -> List[str]:
    """The character that stands for each byte in the vocabulary files (tokenizer.rs:35-49)."""
    table, nxt = [], 256
    for b in range(256):
        if 0x21 <= b <= 0x7E or 0xA1 <= b <= 0xAC or 0xAE <= b <= 0xFF:
            table.append(chr(b))
        else:
            table.append(chr(nxt))
            nxt += 1
    return table


def _class(c: str) -> int:
    if c.isspace():
        return 0
    if c.isalpha():
        return 1
    if c.isnumeric():
        return 2
    return 3


def pre_tokenize(text: str) -> List[str]:
    """The chunks of ``text`` (tokenizer.rs:150-227; equivalent to GPT-2's pattern applied left to right)."""
    out: List[str] = []
    n, i = len(text), 0
    while i < n:
        c = text[i]
        if c == "'":                                             # 1. contractions
            suffix = next((s for s in ("s", "t", "re", "ve", "m", "ll", "d") if text.startswith(s, i + 1)), None)
            if suffix is not None:
                out.append(text[i:i + 1 + len(suffix)])
                i += 1 + len(suffix)
                continue
        start = i + 1 if c == " " else i                         # 2-4. an optional space, then a run of one class
        if start < n and _class(text[start]) != 0:
            cls, end = _class(text[start]), start + 1
            while end < n and _class(text[end]) == cls:
                end += 1
            out.append(text[i:end])
            i = end
            continue
        end = i + 1                                              # 5-6. whitespace
        while end < n and _class(text[end]) == 0:
            end += 1
        if end < n and end - i >= 2:
            end -= 1            # followed by something else: the last one becomes that chunk's leading space
        out.append(text[i:end])
        i = end
    return out


class TokenizerError(ValueError):
    pass


class Tokenizer:
    def __init__(self, vocab: Dict[str, int], merges_text: str):
        b2u = bytes_to_unicode()
        u2b = {c: b for b, c in enumerate(b2u)}
        n = max(vocab.values(), default=-1) + 1
        self.id_to_bytes: List[bytes] = [b""] * n
        for s, i in vocab.items():
            if s == END_OF_TEXT:                                 # special tokens are stored literally
                self.id_to_bytes[i] = s.encode()
                continue
            try:
                self.id_to_bytes[i] = bytes(u2b[c] for c in s)
            except KeyError as e:
                raise TokenizerError(f"tokenizer: vocabulary entry {s!r} holds an unmapped character {e}") from None
        try:
            self.byte_to_id = [vocab[c] for c in b2u]
        except KeyError as e:
            raise TokenizerError(f"tokenizer: no token for the byte written {e}") from None
        self.end_of_text: Optional[int] = vocab.get(END_OF_TEXT)
        #: (left id, right id) -> (rank, merged id)
        self.merges: Dict[Tuple[int, int], Tuple[int, int]] = {}
        rank = 0
        for line in merges_text.splitlines():
            if line.startswith("#version") or not line.strip():
                continue
            parts = line.split(" ")
            if len(parts) != 2:
                raise TokenizerError(f"tokenizer: bad merge line {line!r}")
            a, b = parts
            try:
                self.merges[(vocab[a], vocab[b])] = (rank, vocab[a + b])
            except KeyError as e:
                raise TokenizerError(f"tokenizer: merge token {e} is not in the vocabulary") from None
            rank += 1

    @classmethod
    def from_folder(cls, model_dir: str) -> "Tokenizer":
        """Read ``vocab.json`` and ``merges.txt`` beside the weights (crates/cli/src/main.rs:85-89)."""
        try:
            with open(os.path.join(model_dir, "vocab.json"), encoding="utf-8") as fh:
                vocab = json.load(fh)
            with open(os.path.join(model_dir, "merges.txt"), encoding="utf-8") as fh:
                merges = fh.read()
        except FileNotFoundError as e:
            raise TokenizerError(f"tokenizer: {e.filename}: no such file (a text prompt needs vocab.json and "
                                 f"merges.txt in the model folder; token ids can be given with --prompt-ids)") from None
        except json.JSONDecodeError as e:
            raise TokenizerError(f"tokenizer: vocab.json is not valid JSON ({e})") from None
        return cls(vocab, merges)

    @property
    def vocab_size(self) -> int:
        return len(self.id_to_bytes)

    def _bpe(self, data: bytes, out: List[int]) -> None:
        syms = [self.byte_to_id[b] for b in data]
        while True:
            best = None                                          # (rank, place, merged id): the earliest-learned pair
            for i in range(len(syms) - 1):
                m = self.merges.get((syms[i], syms[i + 1]))
                if m is not None and (best is None or (m[0], i) < best[:2]):
                    best = (m[0], i, m[1])
            if best is None:
                break
            syms[best[1]:best[1] + 2] = [best[2]]
        out.extend(syms)

    def encode(self, text: str) -> List[int]:
        """Token ids of ``text``; ``<|endoftext|>`` in the text becomes its own token (tokenizer.rs:108-120)."""
        ids: List[int] = []
        for k, part in enumerate(text.split(END_OF_TEXT) if self.end_of_text is not None else [text]):
            if k > 0:
                ids.append(self.end_of_text)
            for word in pre_tokenize(part):
                self._bpe(word.encode("utf-8"), ids)
        return ids

    def token_bytes(self, token: int) -> bytes:
        """A token may be part of a multi-byte character: output that streams should collect bytes
        until they are valid UTF-8."""
        return self.id_to_bytes[token] if 0 <= token < len(self.id_to_bytes) else b""

    def decode(self, ids) -> str:
        return b"".join(self.token_bytes(int(i)) for i in ids).decode("utf-8", errors="replace")


def write_byte_tokenizer(model_dir: str, vocab_size: int) -> None:
    """A tokenizer for models with random weights: the 256 byte tokens, no merges, and
    ``<|endoftext|>`` as token 256, so that text can go in and come out of a model that was never
    trained on any.  Needs a vocabulary of at least 257."""
    if vocab_size < 257:
        raise TokenizerError(f"a byte tokenizer needs a vocabulary of at least 257 tokens, the model has {vocab_size}")
    vocab = {c: b for b, c in enumerate(bytes_to_unicode())}
    vocab[END_OF_TEXT] = 256
    with open(os.path.join(model_dir, "vocab.json"), "w", encoding="utf-8") as fh:
        json.dump(vocab, fh, ensure_ascii=False)
    with open(os.path.join(model_dir, "merges.txt"), "w", encoding="utf-8") as fh:
        fh.write("#version: 0.2\n")

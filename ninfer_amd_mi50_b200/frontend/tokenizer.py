"""Byte-level BPE tokenizer read from a HuggingFace ``tokenizer.json``.

What the reference's ``Tokenizer`` does (src/frontend/tokenizer.h:13-47, tokenizer.cpp):
``model.vocab`` and ``model.merges`` (pairs as "a b" strings or two-element lists),
``added_tokens``; text is cut by the Qwen pre-tokenizer pattern (tokenizer.cpp:44-51), every
piece is mapped byte by byte to the GPT-2 printable alphabet and merged greedily by merge
rank; special tokens are the added tokens flagged ``special`` or written like chat markers
(``<|...|>``); the end-of-sequence id is ``<|im_end|>`` if present, else ``<|endoftext|>``
(tokenizer.cpp:268-283).  Generation stops at any special token, as ``Engine::run`` does
(src/runtime/engine.cpp:173).

It sits outside the path from a request's tokens to its next token; the engine takes and
returns token ids, and this is only the convenience around it for ``--prompt`` and
``Ninfer.tokenize / detokenize``.
"""

from __future__ import annotations

import json
from typing import Dict, List, Sequence, Tuple

import regex

PRETOKENIZE = regex.compile(
    r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")


def _byte_alphabet() -> Dict[int, str]:
    """GPT-2's map from byte values to printable characters."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    chars = keep[:]
    n = 0
    for b in range(256):
        if b not in keep:
            keep.append(b)
            chars.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(keep, chars)}


class Tokenizer:
    def __init__(self, tokenizer_json_path: str):
        with open(tokenizer_json_path, "r", encoding="utf-8") as fh:
            data = json.load(fh)
        model = data.get("model") or {}
        vocab = model.get("vocab")
        if not isinstance(vocab, dict) or not vocab:
            raise ValueError(f"{tokenizer_json_path}: no model.vocab")
        self.token_to_id: Dict[str, int] = {t: int(i) for t, i in vocab.items()}
        self.ranks: Dict[Tuple[str, str], int] = {}
        for r, m in enumerate(model.get("merges") or []):
            a, b = m.split(" ", 1) if isinstance(m, str) else (m[0], m[1])
            self.ranks[(a, b)] = r
        self.special: Dict[str, int] = {}
        for t in data.get("added_tokens") or []:
            text, tid = t["content"], int(t["id"])
            self.token_to_id.setdefault(text, tid)
            if t.get("special") or (text.startswith("<|") and text.endswith("|>")):
                self.special[text] = tid
        self.id_to_token: Dict[int, str] = {i: t for t, i in self.token_to_id.items()}
        self.byte_to_char = _byte_alphabet()
        self.char_to_byte = {c: b for b, c in self.byte_to_char.items()}
        self.eos_id = self.special.get("<|im_end|>", self.special.get("<|endoftext|>", -1))
        self._special_split = None
        if self.special:
            alt = "|".join(regex.escape(s) for s in sorted(self.special, key=len, reverse=True))
            self._special_split = regex.compile(f"({alt})")
        self._cache: Dict[str, List[int]] = {}

    @property
    def vocab_size(self) -> int:
        return max(self.id_to_token) + 1

    def is_special(self, token_id: int) -> bool:
        return token_id in self.special.values()

    def stop_ids(self) -> List[int]:
        """Ids at which generation stops: every special token."""
        return sorted(self.special.values())

    # ---- encoding -------------------------------------------------------------------
    def _bpe(self, piece: str) -> List[int]:
        if piece in self._cache:
            return self._cache[piece]
        parts = [self.byte_to_char[b] for b in piece.encode("utf-8")]
        while len(parts) > 1:
            best, at = None, -1
            for i in range(len(parts) - 1):
                r = self.ranks.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            parts[at:at + 2] = [parts[at] + parts[at + 1]]
        ids = []
        for p in parts:
            if p not in self.token_to_id:
                raise ValueError(f"tokenizer: piece {p!r} is not in the vocabulary")
            ids.append(self.token_to_id[p])
        self._cache[piece] = ids
        return ids

    def encode(self, text: str) -> List[int]:
        """Raw text; special tokens written in the text are not recognised."""
        out: List[int] = []
        for piece in PRETOKENIZE.findall(text):
            out += self._bpe(piece)
        return out

    def encode_with_special(self, text: str) -> List[int]:
        """Text in which special tokens (chat markers) stand for themselves."""
        if self._special_split is None:
            return self.encode(text)
        out: List[int] = []
        for part in self._special_split.split(text):
            if part in self.special:
                out.append(self.special[part])
            elif part:
                out += self.encode(part)
        return out

    # ---- decoding -------------------------------------------------------------------
    def decode_bytes(self, ids: Sequence[int], skip_special: bool = False) -> bytes:
        """The bytes the ids stand for.  A multi-byte character may be split between two tokens,
        so text that is printed token by token is cut at the last complete character of these
        bytes, not of each token's own."""
        buf = bytearray()
        for i in ids:
            tok = self.id_to_token.get(int(i))
            if tok is None:
                continue
            if tok in self.special:
                if not skip_special:
                    buf += tok.encode("utf-8")
                continue
            buf += bytes(self.char_to_byte.get(c, ord("?")) for c in tok)
        return bytes(buf)

    def decode(self, ids: Sequence[int], skip_special: bool = False) -> str:
        return self.decode_bytes(ids, skip_special).decode("utf-8", errors="replace")

"""Tokenizer front end, token byte table, incremental detokenisation and stop-string matching.

  * `ByteTokenizer`: a self-contained byte-level tokenizer (256 byte tokens + named specials) used when
    no tokenizer.json is supplied (random-weight benchmarks, tests); `HFTokenizer` wraps the Hugging Face
    `tokenizers` runtime for real checkpoints (reference: crates/sllm-frontend/src/tokenizer.rs).
  * `TokenByteTable`: raw bytes of every token (<= 128 B each), the input of the grammar trie.
  * `IncrementalDetokenizer`: emits only text that can no longer change - an incomplete UTF-8 tail is held
    back until it completes (reference: generation.rs:2360-2392).
  * `IncrementalStopMatcher`: streaming search for up to four stop strings; text that could still become
    a stop string is withheld, and the stop string itself is never emitted (generation.rs:2596-2688).
"""
from __future__ import annotations

from typing import Optional, Sequence

MAX_TOKEN_BYTES = 128


class ByteTokenizer:
    """ids 0..255 are bytes; specials follow.  Deterministic, reversible, no files."""

    SPECIALS = ("<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", "<|fim_prefix|>",
                "<|fim_suffix|>", "<|fim_middle|>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>")

    def __init__(self, vocab_size: int = 256 + 11):
        if vocab_size < 256 + len(self.SPECIALS):
            raise ValueError("vocabulary too small for the byte tokenizer")
        self.vocab_size = vocab_size
        self.special_ids = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.id_to_special = {v: k for k, v in self.special_ids.items()}
        self.eos_token_id = self.special_ids["<|endoftext|>"]
        self.eos_ids = (self.special_ids["<|endoftext|>"], self.special_ids["<|im_end|>"])
        self.identity = "byte-tokenizer-v1"

    def encode(self, text: str, allow_special: bool = True) -> list:
        out = []
        i = 0
        while i < len(text):
            if allow_special and text[i] == "<":
                hit = next((s for s in self.SPECIALS if text.startswith(s, i)), None)
                if hit:
                    out.append(self.special_ids[hit])
                    i += len(hit)
                    continue
            out.extend(text[i].encode("utf-8"))
            i += 1
        return out

    def token_bytes(self, tid: int) -> bytes:
        if 0 <= tid < 256:
            return bytes([tid])
        s = self.id_to_special.get(tid)
        return s.encode() if s else b""

    def is_special(self, tid: int) -> bool:
        return tid >= 256

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = False) -> str:
        b = b"".join(b"" if (skip_special_tokens and self.is_special(t)) else self.token_bytes(t) for t in ids)
        return b.decode("utf-8", errors="replace")

    def pieces(self, ids: Sequence[int]) -> list:
        return [self.token_bytes(t).decode("utf-8", errors="replace") for t in ids]


class HFTokenizer:
    """`tokenizers` runtime wrapper with the same surface as ByteTokenizer."""

    def __init__(self, path_or_json: str, eos_tokens: Sequence[str] = ("<|im_end|>", "<|endoftext|>")):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(path_or_json) if not path_or_json.lstrip().startswith("{") \
            else Tokenizer.from_str(path_or_json)
        self.vocab_size = self.tk.get_vocab_size(with_added_tokens=True)
        self.eos_ids = tuple(i for i in (self.tk.token_to_id(t) for t in eos_tokens) if i is not None)
        self.eos_token_id = self.eos_ids[0] if self.eos_ids else None
        import hashlib
        self.identity = "hf:" + hashlib.sha256(self.tk.to_str().encode()).hexdigest()[:16]
        self._special = {i for t, i in self.tk.get_vocab(with_added_tokens=True).items()
                         if t.startswith("<|") and t.endswith("|>")}
        self._token_bytes: dict = {}

    def encode(self, text: str, allow_special: bool = True) -> list:
        return self.tk.encode(text, add_special_tokens=False).ids

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def is_special(self, tid: int) -> bool:
        return tid in self._special

    def token_bytes(self, tid: int) -> bytes:
        cached = self._token_bytes.get(tid)
        if cached is None:
            cached = self._token_bytes[tid] = self._token_bytes_uncached(tid)      # called once per generated token
        return cached

    def _token_bytes_uncached(self, tid: int) -> bytes:
        tok = self.tk.id_to_token(tid)
        if tok is None:
            return b""
        if tid in self._special:
            return tok.encode()
        # byte-level BPE alphabets map bytes to printable code points; invert that map
        table = _byte_level_inverse()
        try:
            return bytes(table[c] for c in tok)
        except KeyError:
            return tok.replace("▁", " ").encode("utf-8")

    def pieces(self, ids) -> list:
        return [self.tk.id_to_token(t) or "" for t in ids]


_BL = None


def _byte_level_inverse() -> dict:
    global _BL
    if _BL is None:
        bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
        cs = bs[:]
        n = 0
        for b in range(256):
            if b not in bs:
                bs.append(b)
                cs.append(256 + n)
                n += 1
        _BL = {chr(c): b for b, c in zip(bs, cs)}
    return _BL


class TokenByteTable:
    """Raw bytes of every token id (specials have an empty byte string for grammar purposes)."""

    def __init__(self, tokenizer, vocab_size: Optional[int] = None):
        n = vocab_size or tokenizer.vocab_size
        self.bytes = []
        for t in range(n):
            b = b"" if tokenizer.is_special(t) else tokenizer.token_bytes(t)
            if len(b) > MAX_TOKEN_BYTES:
                raise ValueError(f"token {t} is longer than {MAX_TOKEN_BYTES} bytes")
            self.bytes.append(b)

    def __len__(self):
        return len(self.bytes)


def _stable_utf8_prefix(buf: bytes) -> int:
    """Length of the longest prefix of `buf` that does not end inside a UTF-8 sequence."""
    n = len(buf)
    i = n - 1
    back = 0
    while i >= 0 and back < 4 and (buf[i] & 0xC0) == 0x80:
        i -= 1
        back += 1
    if i < 0:
        return n if back == 0 else 0
    lead = buf[i]
    need = 1 if lead < 0x80 else 2 if lead >> 5 == 0b110 else 3 if lead >> 4 == 0b1110 else 4 if lead >> 3 == 0b11110 else 1
    return n if back + 1 >= need else i


class IncrementalDetokenizer:
    def __init__(self, tokenizer, skip_special_tokens: bool = True):
        self.tk = tokenizer
        self.skip_special = skip_special_tokens
        self.pending = b""

    def push(self, tid: int) -> str:
        if self.skip_special and self.tk.is_special(tid):
            return ""
        self.pending += self.tk.token_bytes(tid)
        k = _stable_utf8_prefix(self.pending)
        out, self.pending = self.pending[:k], self.pending[k:]
        return out.decode("utf-8", errors="replace")

    def flush(self) -> str:
        out, self.pending = self.pending, b""
        return out.decode("utf-8", errors="replace")


class IncrementalStopMatcher:
    """Feed text deltas; `push` returns (text safe to publish, stopped)."""

    def __init__(self, stops: Sequence[str]):
        if len(stops) > 4 or any(not s for s in stops) or len(set(stops)) != len(stops):
            raise ValueError("stop must hold 1-4 unique non-empty strings")
        self.stops = list(stops)
        self.held = ""
        self.stopped = False

    def push(self, delta: str):
        if self.stopped:
            return "", True
        if not self.stops:
            return delta, False
        buf = self.held + delta
        first = min((i for i in (buf.find(s) for s in self.stops) if i >= 0), default=-1)
        if first >= 0:
            self.stopped = True
            self.held = ""
            return buf[:first], True
        # keep the longest suffix that is a proper prefix of some stop string
        keep = 0
        for s in self.stops:
            for k in range(min(len(s) - 1, len(buf)), 0, -1):
                if buf.endswith(s[:k]):
                    keep = max(keep, k)
                    break
        self.held = buf[len(buf) - keep:] if keep else ""
        return buf[:len(buf) - keep] if keep else buf, False

    def flush(self) -> str:
        out, self.held = ("" if self.stopped else self.held), ""
        return out

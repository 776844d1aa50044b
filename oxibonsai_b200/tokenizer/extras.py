"""Other tokenizer models: Unigram (Viterbi), WordPiece, character level; ``<0xHH>`` byte fallback; text serialisation
of a BPE vocabulary.

Reference: crates/oxibonsai-tokenizer/src/unigram.rs (best segmentation by log-probability), wordpiece.rs (greedy longest
match with a ``##`` continuation prefix and an unknown token), tokenizer.rs:111-470 (char-level stub, vocabulary and
merges text format) and bpe.rs:142-216 (``<0xHH>`` byte fallback tokens for bytes missing from the vocabulary).
"""
from __future__ import annotations

import math
from typing import Iterable, Sequence


class UnigramTokenizer:
    """Picks the segmentation with the highest total log-probability (Viterbi over byte positions of the text)."""

    def __init__(self, pieces: Sequence[tuple[str, float]], unk_id: int = 0, unk_penalty: float = 10.0):
        self.pieces = [p for p, _ in pieces]
        self.scores = [s for _, s in pieces]
        self.vocab = {p: i for i, p in enumerate(self.pieces)}
        self.unk_id = unk_id
        self.max_len = max((len(p) for p in self.pieces), default=1)
        self._unk_score = min(self.scores, default=0.0) - unk_penalty
        self.vocab_size = len(self.pieces)

    def encode(self, text: str) -> list[int]:
        text = text.replace(" ", "▁")
        n = len(text)
        best = [-math.inf] * (n + 1)
        back: list[tuple[int, int]] = [(0, self.unk_id)] * (n + 1)
        best[0] = 0.0
        for i in range(n):
            if best[i] == -math.inf:
                continue
            matched = False
            for j in range(i + 1, min(n, i + self.max_len) + 1):
                pid = self.vocab.get(text[i:j])
                if pid is not None:
                    matched = matched or j == i + 1
                    s = best[i] + self.scores[pid]
                    if s > best[j]:
                        best[j], back[j] = s, (i, pid)
            if not matched:     # unknown character: one <unk> covering it
                s = best[i] + self._unk_score
                if s > best[i + 1]:
                    best[i + 1], back[i + 1] = s, (i, self.unk_id)
        out, j = [], n
        while j > 0:
            i, pid = back[j]
            out.append(pid)
            j = i
        return out[::-1]

    def decode(self, ids: Iterable[int]) -> str:
        return "".join(self.pieces[i] for i in ids if 0 <= i < len(self.pieces)).replace("▁", " ")

    def token_bytes(self, i: int) -> bytes:
        return self.pieces[i].replace("▁", " ").encode("utf-8") if 0 <= i < len(self.pieces) else b""


class WordPieceTokenizer:
    def __init__(self, vocab: Sequence[str], unk_token: str = "[UNK]", prefix: str = "##", max_chars_per_word: int = 100, lowercase: bool = False):
        self.tokens = list(vocab)
        self.vocab = {t: i for i, t in enumerate(self.tokens)}
        self.unk, self.prefix, self.max_chars, self.lower = unk_token, prefix, max_chars_per_word, lowercase
        self.vocab_size = len(self.tokens)

    def _word(self, w: str) -> list[int]:
        unk = self.vocab.get(self.unk, 0)
        if len(w) > self.max_chars:
            return [unk]
        out, start = [], 0
        while start < len(w):
            end, cur = len(w), None
            while start < end:
                sub = (self.prefix if start > 0 else "") + w[start:end]
                if sub in self.vocab:
                    cur = self.vocab[sub]
                    break
                end -= 1
            if cur is None:
                return [unk]
            out.append(cur)
            start = end
        return out

    def encode(self, text: str) -> list[int]:
        if self.lower:
            text = text.lower()
        words, cur = [], ""
        for ch in text:
            if ch.isspace():
                if cur:
                    words.append(cur)
                cur = ""
            elif not ch.isalnum():
                if cur:
                    words.append(cur)
                words.append(ch)
                cur = ""
            else:
                cur += ch
        if cur:
            words.append(cur)
        return [i for w in words for i in self._word(w)]

    def decode(self, ids: Iterable[int]) -> str:
        out = ""
        for i in ids:
            t = self.tokens[i] if 0 <= i < len(self.tokens) else self.unk
            out += t[len(self.prefix):] if t.startswith(self.prefix) else ((" " if out else "") + t)
        return out

    def token_bytes(self, i: int) -> bytes:
        t = self.tokens[i] if 0 <= i < len(self.tokens) else ""
        return (t[len(self.prefix):] if t.startswith(self.prefix) else " " + t).encode("utf-8")


class CharTokenizer:
    """One id per Unicode code point seen at construction; unknown characters map to id 0."""

    def __init__(self, alphabet: Iterable[str]):
        self.chars = ["�"] + sorted(set(alphabet))
        self.vocab = {c: i for i, c in enumerate(self.chars)}
        self.vocab_size = len(self.chars)

    def encode(self, text: str) -> list[int]:
        return [self.vocab.get(c, 0) for c in text]

    def decode(self, ids: Iterable[int]) -> str:
        return "".join(self.chars[i] if 0 <= i < len(self.chars) else "�" for i in ids)

    def token_bytes(self, i: int) -> bytes:
        return self.chars[i].encode("utf-8") if 0 <= i < len(self.chars) else b""


# ---- byte fallback ----------------------------------------------------------------------------------------------------------
def byte_fallback_token(b: int) -> str:
    return f"<0x{b:02X}>"


def parse_byte_fallback(token: str) -> int | None:
    if len(token) == 6 and token.startswith("<0x") and token.endswith(">"):
        try:
            return int(token[3:5], 16)
        except ValueError:
            return None
    return None


def encode_with_byte_fallback(text: str, vocab: dict[str, int], unk_id: int = 0) -> list[int]:
    """Character-level lookup; characters missing from ``vocab`` become their UTF-8 bytes as ``<0xHH>`` tokens."""
    out = []
    for ch in text:
        if ch in vocab:
            out.append(vocab[ch])
        else:
            for b in ch.encode("utf-8"):
                out.append(vocab.get(byte_fallback_token(b), unk_id))
    return out


def decode_with_byte_fallback(ids: Iterable[int], id_to_token: dict[int, str]) -> str:
    buf = bytearray()
    for i in ids:
        t = id_to_token.get(int(i), "")
        b = parse_byte_fallback(t)
        buf += bytes([b]) if b is not None else t.encode("utf-8")
    return buf.decode("utf-8", errors="replace")


# ---- text serialisation of a BPE model ---------------------------------------------------------------------------------------
def save_bpe_text(tokenizer, path: str) -> None:
    """``#vocab`` section (token<TAB>id), ``#merges`` section (left<SPACE>right), ``#special`` section."""
    with open(path, "w", encoding="utf-8") as f:
        f.write("#vocab\n")
        for t, i in sorted(tokenizer.vocab.items(), key=lambda kv: kv[1]):
            f.write(f"{t}\t{i}\n")
        f.write("#merges\n")
        inv = {i: t for t, i in tokenizer.vocab.items()}
        for a, b, _ in tokenizer.merges:
            f.write(f"{inv[a]} {inv[b]}\n")
        f.write("#special\n")
        for t, i in tokenizer.special.items():
            f.write(f"{t}\t{i}\n")


def load_bpe_text(path: str):
    from . import BpeTokenizer
    vocab, merges, special, section = {}, [], {}, None
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.rstrip("\n")
            if line in ("#vocab", "#merges", "#special"):
                section = line
            elif not line:
                continue
            elif section == "#merges":
                a, b = line.split(" ", 1)
                merges.append((a, b))
            else:
                t, i = line.rsplit("\t", 1)
                (vocab if section == "#vocab" else special)[t] = int(i)
    return BpeTokenizer(vocab, merges, special)

"""Tokenizers: native byte-level BPE (C++ merge engine), HF ``tokenizers`` bridge, byte fallback, chat templates.

Reference: ``OxiTokenizer`` with BPE / byte fallback / HF ``tokenizer.json`` loading, streaming UTF-8 decoding, a BPE
trainer and five chat templates (crates/oxibonsai-tokenizer/src/tokenizer.rs:111-470, bpe.rs, hf_format.rs, streaming.rs,
trainer.rs, chat_templates.rs:65-76) and the runtime bridges ``TokenizerBridge`` / ``NativeTokenizerBridge``
(crates/oxibonsai-runtime/src/tokenizer_bridge.rs:12-200, native_tokenizer.rs).
"""
from __future__ import annotations

import ctypes as C
import json
from collections import Counter
from functools import lru_cache
from typing import Iterable, Sequence

import numpy as np

from .. import _native

_GPT2_SPLIT = r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"""


@lru_cache(maxsize=1)
def bytes_to_unicode() -> dict[int, str]:
    """The reversible byte <-> printable-character map of byte-level BPE vocabularies."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


def _declare():
    lib = _native.host()
    if "bbpe_new" not in lib._declared:
        _native.declare(lib, {"bbpe_new": (C.c_void_p, [C.c_void_p, C.c_uint64]), "bbpe_free": (None, [C.c_void_p]),
                              "bbpe_merge": (C.c_uint64, [C.c_void_p, C.c_void_p, C.c_uint64]),
                              "bbpe_encode": (C.c_uint64, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_uint64])})
        lib._declared.add("bbpe_new")
    return lib


class StreamingDecoder:
    """Turns a stream of token byte strings into text without ever splitting a UTF-8 sequence."""

    def __init__(self):
        self._buf = b""

    def push(self, data: bytes) -> str:
        self._buf += data
        # longest prefix that is complete UTF-8
        end = len(self._buf)
        for back in range(1, min(4, end) + 1):
            b = self._buf[end - back]
            if b & 0xC0 == 0x80:
                continue
            need = 1 if b < 0x80 else (2 if b >> 5 == 0b110 else (3 if b >> 4 == 0b1110 else (4 if b >> 3 == 0b11110 else 1)))
            if need > back:
                end -= back
            break
        out, self._buf = self._buf[:end], self._buf[end:]
        return out.decode("utf-8", errors="replace")

    def flush(self) -> str:
        out, self._buf = self._buf, b""
        return out.decode("utf-8", errors="replace")


class ByteTokenizer:
    """ids 0..255 are bytes; useful for synthetic checkpoints and tests."""

    vocab_size = 256

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids: Iterable[int]) -> str:
        return bytes(i & 0xFF for i in ids).decode("utf-8", errors="replace")

    def token_bytes(self, i: int) -> bytes:
        return bytes([i & 0xFF])


class BpeTokenizer:
    """Byte-level BPE with the merge loop in C++."""

    def __init__(self, vocab: dict[str, int], merges: Sequence[tuple[str, str]], special_tokens: dict[str, int] | None = None,
                 split_pattern: str = _GPT2_SPLIT):
        import regex
        self.vocab = dict(vocab)
        self.special = dict(special_tokens or {})
        # the token that ends an assistant turn, where the vocabulary names one (chat models end turns with <|im_end|> /
        # <|eot_id|>, base models documents with <|endoftext|> / </s>)
        self.eos_token_id: int | None = next((self.special[n] for n in ("<|im_end|>", "<|eot_id|>", "<|endoftext|>", "</s>", "<EOS>") if n in self.special), None)
        self.bos_token_id: int | None = next((self.special[n] for n in ("<|begin_of_text|>", "<s>", "<BOS>") if n in self.special), None)
        self.id_to_token = {i: t for t, i in {**self.vocab, **self.special}.items()}
        self.vocab_size = max(self.id_to_token) + 1 if self.id_to_token else 0
        self._split = regex.compile(split_pattern)
        self._special_re = regex.compile("|".join(regex.escape(s) for s in sorted(self.special, key=len, reverse=True))) if self.special else None
        self._b2u = bytes_to_unicode()
        self._u2b = {u: b for b, u in self._b2u.items()}
        self._byte_id = [self.vocab.get(self._b2u[b], -1) for b in range(256)]
        self._byte_id_arr = np.asarray(self._byte_id, dtype=np.int32)
        trip = []
        for a, b in merges:
            ia, ib, im = self.vocab.get(a), self.vocab.get(b), self.vocab.get(a + b)
            if ia is not None and ib is not None and im is not None:
                trip.append((ia, ib, im))
        self.merges = trip
        arr = np.asarray(trip, dtype=np.uint32).reshape(-1, 3) if trip else np.zeros((0, 3), dtype=np.uint32)
        self._lib = _declare()
        self._h = self._lib.bbpe_new(arr.ctypes.data if len(arr) else None, len(arr))

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.bbpe_free(self._h)
            self._h = None

    @classmethod
    def from_hf_json(cls, path: str) -> "BpeTokenizer":
        """Loads a Hugging Face ``tokenizer.json`` with a byte-level BPE model."""
        with open(path, encoding="utf-8") as f:
            j = json.load(f)
        model = j["model"]
        if model.get("type", "BPE") != "BPE":
            raise ValueError(f"unsupported tokenizer model type {model.get('type')}")
        merges = [tuple(m.split(" ", 1)) if isinstance(m, str) else tuple(m) for m in model.get("merges", [])]
        special = {t["content"]: t["id"] for t in j.get("added_tokens", [])}

        def split_pattern(node) -> str | None:
            """The regular expression of the file's ``Split`` pre-tokenizer (Qwen, Llama-3 ... ship their own)."""
            if isinstance(node, dict):
                if node.get("type") == "Split" and isinstance(node.get("pattern"), dict) and "Regex" in node["pattern"]:
                    return node["pattern"]["Regex"]
                for v in node.values():
                    found = split_pattern(v)
                    if found:
                        return found
            elif isinstance(node, list):
                for v in node:
                    found = split_pattern(v)
                    if found:
                        return found
            return None
        pattern = split_pattern(j.get("pre_tokenizer"))
        tok = None
        if pattern:
            try:
                import regex
                regex.compile(pattern)
                tok = cls(model["vocab"], merges, special, pattern)
            except Exception:  # noqa: BLE001 - a dialect the regex module does not take: the GPT-2 pattern is the fallback
                tok = None
        tok = tok or cls(model["vocab"], merges, special)

        def normal_form(node) -> str | None:
            """Unicode normalisation the file asks for (Qwen: NFC), applied to plain text before splitting."""
            if isinstance(node, dict):
                if node.get("type") in ("NFC", "NFD", "NFKC", "NFKD"):
                    return node["type"]
                return next((f for f in (normal_form(v) for v in node.values()) if f), None)
            if isinstance(node, list):
                return next((f for f in (normal_form(v) for v in node) if f), None)
            return None
        tok.normal_form = normal_form(j.get("normalizer"))
        return tok

    QWEN_SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")

    @classmethod
    def from_gguf(cls, gguf) -> "BpeTokenizer":
        """The byte-level BPE vocabulary a GGUF file carries in its metadata (``tokenizer.ggml.model = "gpt2"``:
        ``tokens``, ``merges``, ``token_type`` with 3 = control and 4 = user-defined tokens, ``pre`` naming the split
        pattern, ``bos`` / ``eos_token_id``).  ``gguf``: a path or an open ``GgufFile``.  The reference defines these keys
        (crates/oxibonsai-core/src/gguf/tensor_info.rs:203-206) and loads tokenizers from ``tokenizer.json`` only; with this
        a checkpoint that embeds its vocabulary needs no side file."""
        if isinstance(gguf, (str, bytes)) or hasattr(gguf, "__fspath__"):
            from ..core import GgufFile
            gguf = GgufFile.open(str(gguf))
        md = gguf.metadata
        kind = md.get("tokenizer.ggml.model")
        if kind != "gpt2":
            raise ValueError(f"the file embeds no byte-level BPE vocabulary (tokenizer.ggml.model = {kind!r})")
        tokens = list(md.get("tokenizer.ggml.tokens") or [])
        if not tokens:
            raise ValueError("tokenizer.ggml.tokens is empty")
        types = list(md.get("tokenizer.ggml.token_type") or [])
        vocab, special = {}, {}
        for i, t in enumerate(tokens):
            if i < len(types) and types[i] in (3, 4):
                special[t] = i
            else:
                vocab[t] = i
        merges = [tuple(m.split(" ", 1)) for m in md.get("tokenizer.ggml.merges") or [] if " " in m]
        pre = str(md.get("tokenizer.ggml.pre") or "")
        tok = cls(vocab, merges, special, cls.QWEN_SPLIT if pre.startswith("qwen") else _GPT2_SPLIT)
        tok.normal_form = "NFC" if pre.startswith("qwen") else None
        if md.get("tokenizer.ggml.eos_token_id") is not None:
            tok.eos_token_id = int(md["tokenizer.ggml.eos_token_id"])
        if md.get("tokenizer.ggml.bos_token_id") is not None:
            tok.bos_token_id = int(md["tokenizer.ggml.bos_token_id"])
        return tok

    def _encode_piece(self, piece: str) -> list[int]:
        raw = piece.encode("utf-8")
        ids = np.fromiter((self._byte_id[b] for b in raw), dtype=np.int64, count=len(raw))
        if (ids < 0).any():
            ids = ids[ids >= 0]
        buf = ids.astype(np.uint32)
        if buf.size <= 1:
            return buf.tolist()
        n = self._lib.bbpe_merge(self._h, buf.ctypes.data, buf.size)
        return buf[:n].tolist()

    def encode(self, text: str, allow_special: bool = True) -> list[int]:
        out: list[int] = []
        segments: list[tuple[str, bool]] = []
        if allow_special and self._special_re is not None:
            pos = 0
            for m in self._special_re.finditer(text):
                if m.start() > pos:
                    segments.append((text[pos:m.start()], False))
                segments.append((m.group(), True))
                pos = m.end()
            if pos < len(text):
                segments.append((text[pos:], False))
        else:
            segments = [(text, False)]
        form = getattr(self, "normal_form", None)
        for seg, is_special in segments:
            if is_special:
                out.append(self.special[seg])
            else:
                if form:
                    import unicodedata
                    seg = unicodedata.normalize(form, seg)
                out.extend(self._encode_plain(seg))
        return out

    def _encode_plain(self, seg: str) -> list[int]:
        """Splits a segment without special tokens and merges all of its pieces in one native call."""
        pieces = self._split.findall(seg) if not self._split.groups else [m.group() for m in self._split.finditer(seg)]
        if not pieces:
            return []
        raw = "".join(pieces).encode("utf-8")                      # == seg for a pattern that tiles the text (the usual ones do)
        lens = list(map(len, pieces))
        if sum(lens) != len(raw):                                   # not ASCII: lengths in bytes
            lens = list(map(len, map(str.encode, pieces)))
        ends = np.cumsum(np.asarray(lens, dtype=np.uint64), dtype=np.uint64)
        buf = np.empty(max(1, len(raw)), dtype=np.uint32)
        n = self._lib.bbpe_encode(self._h, raw, ends.ctypes.data, len(ends), self._byte_id_arr.ctypes.data, buf.ctypes.data, buf.size)
        return buf[:n].tolist()

    def token_bytes(self, i: int) -> bytes:
        t = self.id_to_token.get(int(i))
        if t is None:
            return b""
        if t in self.special:
            return t.encode("utf-8")
        return bytes(self._u2b.get(ch, ord("?")) for ch in t)

    def decode(self, ids: Iterable[int], skip_special: bool = False) -> str:
        data = b"".join(b"" if (skip_special and self.id_to_token.get(int(i)) in self.special) else self.token_bytes(i) for i in ids)
        return data.decode("utf-8", errors="replace")

    def encode_batch(self, texts: Sequence[str]) -> list[list[int]]:
        return [self.encode(t) for t in texts]


def train_bpe(corpus: Iterable[str], vocab_size: int, special_tokens: Sequence[str] = ()) -> BpeTokenizer:
    """Small reference trainer: byte-level pre-tokenisation, then greedy most-frequent-pair merges."""
    import regex
    split = regex.compile(_GPT2_SPLIT)
    b2u = bytes_to_unicode()
    words: Counter = Counter()
    for text in corpus:
        for piece in split.findall(text):
            words[tuple(b2u[b] for b in piece.encode("utf-8"))] += 1
    vocab = {b2u[b]: b for b in range(256)}
    merges: list[tuple[str, str]] = []
    from ._merge_learner import MergeLearner
    learner = MergeLearner(words, make=lambda a, b, _i: a + b, tie=lambda pair: pair)       # ties: the larger pair wins
    while len(vocab) < vocab_size - len(special_tokens):
        found = learner.best()
        if found is None or found[1] < 2:
            break
        a, b = found[0]
        learner.merge(found[0])
        merges.append((a, b))
        vocab[a + b] = len(vocab)
    special = {s: len(vocab) + i for i, s in enumerate(special_tokens)}
    return BpeTokenizer(vocab, merges, special)


class HfTokenizerBridge:
    """Bridge over the Hugging Face ``tokenizers`` library (the same Rust tokenizer the reference links)."""

    def __init__(self, path: str):
        from tokenizers import Tokenizer
        self._t = Tokenizer.from_file(path)
        self.vocab_size = self._t.get_vocab_size()
        # Byte-level models spell every token in the 256-character byte alphabet; a token may be a fragment of a UTF-8
        # character, which ``decode`` would turn into U+FFFD.  Streaming needs the real bytes.
        spec = json.loads(self._t.to_str())

        def byte_level(node) -> bool:
            if isinstance(node, dict):
                return node.get("type") == "ByteLevel" or any(byte_level(v) for v in node.values())
            return isinstance(node, list) and any(byte_level(v) for v in node)
        self._u2b = {u: b for b, u in bytes_to_unicode().items()} if byte_level(spec.get("decoder")) else None
        self._special = {t["id"] for t in spec.get("added_tokens", []) if t.get("special")}

    def encode(self, text: str) -> list[int]:
        return self._t.encode(text, add_special_tokens=False).ids

    def decode(self, ids: Iterable[int]) -> str:
        return self._t.decode(list(ids), skip_special_tokens=False)

    def token_bytes(self, i: int) -> bytes:
        i = int(i)
        if self._u2b is not None and i not in self._special:
            piece = self._t.id_to_token(i)
            if piece is not None:
                try:
                    return bytes(self._u2b[ch] for ch in piece)
                except KeyError:            # an added token written in plain text
                    return piece.encode("utf-8")
        return self._t.decode([i], skip_special_tokens=False).encode("utf-8")


# ---- chat templates -------------------------------------------------------------------------------------
def chat_prompt(messages: Sequence[dict], template: str = "chatml", add_generation_prompt: bool = True) -> str:
    """Renders ``[{role, content}, ...]`` with one of: chatml / qwen, llama3, mistral, gemma."""
    t = template.lower()
    if t in ("chatml", "qwen"):
        s = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in messages)
        return s + ("<|im_start|>assistant\n" if add_generation_prompt else "")
    if t == "llama3":
        s = "<|begin_of_text|>" + "".join(f"<|start_header_id|>{m['role']}<|end_header_id|>\n\n{m['content']}<|eot_id|>" for m in messages)
        return s + ("<|start_header_id|>assistant<|end_header_id|>\n\n" if add_generation_prompt else "")
    if t == "mistral":
        s, sys_ = "<s>", ""
        for m in messages:
            if m["role"] == "system":
                sys_ = m["content"] + "\n\n"
            elif m["role"] == "user":
                s += f"[INST] {sys_}{m['content']} [/INST]"
                sys_ = ""
            else:
                s += f" {m['content']}</s>"
        return s
    if t == "gemma":
        s = "<bos>" + "".join(f"<start_of_turn>{'model' if m['role'] == 'assistant' else 'user'}\n{m['content']}<end_of_turn>\n" for m in messages)
        return s + ("<start_of_turn>model\n" if add_generation_prompt else "")
    raise ValueError(f"unknown chat template {template!r}")


def load_tokenizer(path: str | None, kind: str = "auto", model_path: str | None = None):
    """``kind``: auto / native / hf / bytes.  ``auto`` prefers the native BPE for tokenizer.json files.  Without a tokenizer
    file, a vocabulary embedded in the checkpoint at ``model_path`` is used when there is one; raw bytes are the last resort."""
    if kind == "bytes":
        return ByteTokenizer()
    if path is None:
        if model_path is not None:
            try:
                return BpeTokenizer.from_gguf(model_path)
            except Exception:  # noqa: BLE001 - no embedded vocabulary (or not a GGUF file)
                pass
        return ByteTokenizer()
    if str(path).endswith(".gguf"):
        return BpeTokenizer.from_gguf(path)
    if kind in ("auto", "native"):
        try:
            return BpeTokenizer.from_hf_json(path)
        except Exception:
            if kind == "native":
                raise
    return HfTokenizerBridge(path)

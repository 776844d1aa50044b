"""Tokenizer toolkit: vocabulary with special tokens, chat-template families with a small template evaluator, text
normalisation, batch encoding with truncation and padding, a configurable BPE trainer with statistics, a serialisable
tokenizer state, and a token-level streaming decoder.

Reference: crates/oxibonsai-tokenizer - vocab.rs (``Vocabulary``), chat_templates.rs (ChatML / Llama-3 / Mistral / Gemma /
Qwen as Jinja-like templates with ``{% for message in messages %}``, ``{{ role }}``, ``{{ content }}`` and
``{% if role == "user" %} .. {% else %} .. {% endif %}``; generation prompts; ``infer_from_name``), utils.rs
(``TextNormalizer``: lowercase -> strip accents -> strip -> collapse; ``ChatTemplate.extract_user_message``; ``BatchEncoder``
with truncation side and padding strategy, attention masks), trainer.rs (``TrainerConfig``: vocabulary size, minimum
pair frequency, special tokens BOS / EOS / PAD / UNK at ids 0-3; ``TrainingStats``; ``merges_to_text``), serialization.rs
(``TokenizerState``: id -> token, merge triples, special tokens; base64 for token bytes), streaming.rs (token-level
streaming decoder with pending bytes, strict and lossy finish).
"""
from __future__ import annotations

import base64
import json
import re
import unicodedata
from collections import Counter
from dataclasses import dataclass, field
from enum import Enum
from typing import Iterable, Iterator, Sequence


# ---- vocabulary ---------------------------------------------------------------------------------------------------------------
class Vocabulary:
    """Token string <-> id, with a set of ids marked special."""

    def __init__(self):
        self._tok2id: dict[str, int] = {}
        self._id2tok: dict[int, str] = {}
        self._special: set[int] = set()

    def insert(self, token: str, token_id: int) -> None:
        old = self._tok2id.get(token)
        if old is not None and old != token_id:
            self._id2tok.pop(old, None)
        self._tok2id[token] = token_id
        self._id2tok[token_id] = token

    def add_special(self, token: str, token_id: int) -> None:
        self.insert(token, token_id)
        self._special.add(token_id)

    def get_id(self, token: str) -> int | None:
        return self._tok2id.get(token)

    def get_token(self, token_id: int) -> str | None:
        return self._id2tok.get(token_id)

    def size(self) -> int:
        return len(self._tok2id)

    __len__ = size

    def is_empty(self) -> bool:
        return not self._tok2id

    def is_special_token(self, token: str) -> bool:
        return self._tok2id.get(token) in self._special

    def is_special_id(self, token_id: int) -> bool:
        return token_id in self._special

    def __iter__(self) -> Iterator[tuple[str, int]]:
        return iter(sorted(self._tok2id.items(), key=lambda kv: kv[1]))

    def to_json(self) -> str:
        return json.dumps({"vocab": dict(iter(self)), "special": sorted(self._special)}, ensure_ascii=False)

    @classmethod
    def from_json(cls, text: str) -> "Vocabulary":
        doc = json.loads(text)
        table = doc["vocab"] if isinstance(doc, dict) and "vocab" in doc else doc          # a bare {token: id} map is accepted
        v = cls()
        for tok, i in table.items():
            v.insert(tok, int(i))
        for i in (doc.get("special", []) if isinstance(doc, dict) else []):
            v._special.add(int(i))
        return v


# ---- chat templates -----------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class ChatMessage:
    role: str
    content: str

    @classmethod
    def user(cls, content: str) -> "ChatMessage":
        return cls("user", content)

    @classmethod
    def assistant(cls, content: str) -> "ChatMessage":
        return cls("assistant", content)

    @classmethod
    def system(cls, content: str) -> "ChatMessage":
        return cls("system", content)


_FOR = re.compile(r"\{%\s*for\s+message\s+in\s+messages\s*%\}(.*?)\{%\s*endfor\s*%\}", re.S)
_IF = re.compile(r"\{%\s*if\s+role\s*(==|!=)\s*\"([^\"]*)\"\s*%\}(.*?)(?:\{%\s*else\s*%\}(.*?))?\{%\s*endif\s*%\}", re.S)


def render_template(template: str, messages: Sequence[tuple[str, str]]) -> str:
    """Evaluates the template subset the chat families need: one loop over the messages, ``{{ role }}`` /
    ``{{ content }}`` substitution and ``{% if role == "x" %} a {% else %} b {% endif %}`` inside the loop.  Text outside the
    loop is copied once."""
    def body(text: str, role: str, content: str) -> str:
        def pick(m: re.Match) -> str:
            hit = (role == m.group(2)) == (m.group(1) == "==")
            return m.group(3) if hit else (m.group(4) or "")
        text = _IF.sub(pick, text)
        # substitute in one pass so that a message containing "{{ role }}" is not expanded again
        return re.sub(r"\{\{\s*(role|content)\s*\}\}", lambda m: role if m.group(1) == "role" else content, text)
    return _FOR.sub(lambda m: "".join(body(m.group(1), r, c) for r, c in messages), template)


class ChatTemplateKind(Enum):
    CHATML = "chatml"
    LLAMA3 = "llama3"
    MISTRAL = "mistral"
    GEMMA = "gemma"
    QWEN = "qwen"

    def template(self) -> str:
        return _TEMPLATES[self]

    def generation_prompt(self) -> str:
        return {ChatTemplateKind.CHATML: "<|im_start|>assistant\n", ChatTemplateKind.QWEN: "<|im_start|>assistant\n",
                ChatTemplateKind.LLAMA3: "<|start_header_id|>assistant<|end_header_id|>\n\n", ChatTemplateKind.MISTRAL: "",
                ChatTemplateKind.GEMMA: "<start_of_turn>model\n"}[self]

    def render(self, messages: Sequence[ChatMessage]) -> str:
        return render_template(self.template(), [(m.role, m.content) for m in messages])

    def render_with_generation_prompt(self, messages: Sequence[ChatMessage]) -> str:
        return self.render(messages) + self.generation_prompt()

    def encode(self, tokenizer, messages: Sequence[ChatMessage], add_generation_prompt: bool = True) -> list[int]:
        return tokenizer.encode(self.render_with_generation_prompt(messages) if add_generation_prompt else self.render(messages))

    @classmethod
    def all(cls) -> list["ChatTemplateKind"]:
        return list(cls)

    @classmethod
    def infer_from_name(cls, name: str) -> "ChatTemplateKind | None":
        n = name.lower()
        if "llama-3" in n or "llama3" in n:
            return cls.LLAMA3
        for key, kind in (("mistral", cls.MISTRAL), ("gemma", cls.GEMMA), ("qwen", cls.QWEN), ("chatml", cls.CHATML)):
            if key in n:
                return kind
        return None


_CHATML = "{% for message in messages %}<|im_start|>{{ role }}\n{{ content }}<|im_end|>\n{% endfor %}"
_TEMPLATES = {
    ChatTemplateKind.CHATML: _CHATML,
    ChatTemplateKind.QWEN: _CHATML,
    ChatTemplateKind.LLAMA3: "<|begin_of_text|>{% for message in messages %}<|start_header_id|>{{ role }}<|end_header_id|>\n\n{{ content }}<|eot_id|>{% endfor %}",
    ChatTemplateKind.MISTRAL: '{% for message in messages %}{% if role == "user" %}<s>[INST] {{ content }} [/INST]{% else %} {{ content }}</s>{% endif %}{% endfor %}',
    ChatTemplateKind.GEMMA: "{% for message in messages %}<start_of_turn>{{ role }}\n{{ content }}<end_of_turn>\n{% endfor %}",
}


class ChatTemplate:
    """A user-supplied template in the same subset."""

    def __init__(self, template: str):
        self.template = template

    @classmethod
    def chatml(cls) -> "ChatTemplate":
        return cls(_CHATML)

    @classmethod
    def llama3(cls) -> "ChatTemplate":
        return cls(_TEMPLATES[ChatTemplateKind.LLAMA3])

    def format(self, messages: Sequence[tuple[str, str]]) -> str:
        return render_template(self.template, list(messages))

    @staticmethod
    def extract_user_message(prompt: str) -> str | None:
        """The content of the last ``<|im_start|>user ... <|im_end|>`` block of a ChatML prompt."""
        start = prompt.rfind("<|im_start|>user\n")
        if start < 0:
            return None
        start += len("<|im_start|>user\n")
        end = prompt.find("<|im_end|>", start)
        return prompt[start:end] if end >= 0 else None


# ---- normalisation ------------------------------------------------------------------------------------------------------------
@dataclass
class TextNormalizer:
    lowercase: bool = False
    strip_accents: bool = False
    strip_whitespace: bool = True
    collapse_whitespace: bool = True

    @classmethod
    def lowercase_only(cls) -> "TextNormalizer":
        return cls(True, False, False, False)

    @classmethod
    def whitespace_only(cls) -> "TextNormalizer":
        return cls(False, False, True, True)

    def normalize(self, text: str) -> str:
        if self.lowercase:
            text = text.lower()          # Unicode-aware (the reference lowercases ASCII only: "Û" would survive as "U" after accent stripping)
        if self.strip_accents:
            text = "".join(c for c in unicodedata.normalize("NFD", text) if not unicodedata.combining(c))
        if self.strip_whitespace:
            text = text.strip()
        if self.collapse_whitespace:
            text = re.sub(r"\s+", " ", text)
        return text


# ---- batches ------------------------------------------------------------------------------------------------------------------
class TruncationSide(Enum):
    LEFT = "left"
    RIGHT = "right"


@dataclass(frozen=True)
class PaddingStrategy:
    fixed: int | None = None             # None: pad to the longest sequence of the batch

    @classmethod
    def longest(cls) -> "PaddingStrategy":
        return cls(None)

    @classmethod
    def to(cls, n: int) -> "PaddingStrategy":
        return cls(int(n))


@dataclass
class BatchEncoding:
    input_ids: list[list[int]]
    attention_mask: list[list[int]]
    lengths: list[int]

    def batch_size(self) -> int:
        return len(self.input_ids)

    def max_seq_len(self) -> int:
        return max((len(r) for r in self.input_ids), default=0)

    def is_padded(self) -> bool:
        return any(0 in m for m in self.attention_mask)


class BatchEncoder:
    def __init__(self, tokenizer, pad_id: int = 0):
        self.tokenizer, self.pad_id = tokenizer, pad_id
        self.max_length: int | None = None
        self.truncation = TruncationSide.RIGHT
        self.padding: PaddingStrategy | None = None
        self.pad_left = False

    def with_max_length(self, n: int) -> "BatchEncoder":
        self.max_length = n
        return self

    def with_truncation(self, side: TruncationSide) -> "BatchEncoder":
        self.truncation = side
        return self

    def with_padding(self, strategy: PaddingStrategy, left: bool = False) -> "BatchEncoder":
        """``left``: pad in front (what a decoder-only model wants for batched generation)."""
        self.padding, self.pad_left = strategy, left
        return self

    def encode_batch(self, texts: Sequence[str]) -> BatchEncoding:
        rows = []
        for t in texts:
            ids = list(self.tokenizer.encode(t))
            if self.max_length is not None and len(ids) > self.max_length:
                ids = ids[-self.max_length:] if self.truncation is TruncationSide.LEFT else ids[:self.max_length]
            rows.append(ids)
        lengths = [len(r) for r in rows]
        if self.padding is None:
            return BatchEncoding(rows, [[1] * n for n in lengths], lengths)
        width = self.padding.fixed if self.padding.fixed is not None else max(lengths, default=0)
        ids_out, mask_out = [], []
        for r in rows:
            r = r[:width] if self.truncation is TruncationSide.RIGHT else r[max(0, len(r) - width):]
            pad = [self.pad_id] * (width - len(r))
            ids_out.append(pad + r if self.pad_left else r + pad)
            mask_out.append([0] * len(pad) + [1] * len(r) if self.pad_left else [1] * len(r) + [0] * len(pad))
        return BatchEncoding(ids_out, mask_out, [min(n, width) for n in lengths])


# ---- BPE trainer --------------------------------------------------------------------------------------------------------------
SPECIAL_TOKENS = ("<BOS>", "<EOS>", "<PAD>", "<UNK>")


@dataclass
class TrainerConfig:
    vocab_size: int = 512
    min_frequency: int = 2
    add_special_tokens: bool = False      # BOS / EOS / PAD / UNK at ids 0..3, byte tokens from id 4
    byte_level: bool = True               # pre-tokenise on white-space boundaries (GPT-2 style) before merging
    progress_interval: int | None = None

    def with_min_frequency(self, n: int) -> "TrainerConfig":
        self.min_frequency = n
        return self

    def with_special_tokens(self, on: bool = True) -> "TrainerConfig":
        self.add_special_tokens = on
        return self


class TrainerError(ValueError):
    pass


@dataclass
class MergeRule:
    left: int
    right: int
    merged: int
    frequency: int


@dataclass
class TrainingStats:
    initial_vocab_size: int
    final_vocab_size: int
    num_merges_performed: int
    num_merges_skipped: int
    corpus_size_chars: int
    unique_words: int

    def summary(self) -> str:
        return (f"BPE training: {self.initial_vocab_size} -> {self.final_vocab_size} tokens | {self.num_merges_performed} merges applied, "
                f"{self.num_merges_skipped} skipped | corpus {self.corpus_size_chars} bytes, {self.unique_words} unique words")


@dataclass
class TrainedTokenizer:
    vocab: dict[int, bytes]               # id -> the bytes the token stands for
    merges: list[MergeRule]
    special_tokens: dict[str, int]
    stats: TrainingStats

    def vocab_size(self) -> int:
        return len(self.vocab) + len(self.special_tokens)

    def merges_to_text(self) -> str:
        """One ``left right`` line per merge, tokens in the byte-to-unicode alphabet of GPT-2 style ``merges.txt`` files."""
        from . import bytes_to_unicode
        b2u = bytes_to_unicode()
        show = lambda i: "".join(b2u[b] for b in self.vocab[i])
        return "".join(f"{show(m.left)} {show(m.right)}\n" for m in self.merges)

    def to_tokenizer(self):
        """The trained model as a :class:`~oxibonsai_b200.tokenizer.BpeTokenizer` (merge loop in C++)."""
        from . import BpeTokenizer, bytes_to_unicode
        b2u = bytes_to_unicode()
        name = lambda i: "".join(b2u[b] for b in self.vocab[i])
        vocab = {name(i): i for i in self.vocab}
        merges = [(name(m.left), name(m.right)) for m in self.merges]
        return BpeTokenizer(vocab, merges, dict(self.special_tokens))


class BpeTrainer:
    def __init__(self, config: TrainerConfig | None = None):
        self.config = config or TrainerConfig()

    @classmethod
    def default_config(cls) -> "BpeTrainer":
        return cls(TrainerConfig())

    def train(self, corpus: Iterable[str]) -> TrainedTokenizer:
        cfg = self.config
        base = 4 if cfg.add_special_tokens else 0
        if cfg.vocab_size < base + 256:
            raise TrainerError(f"vocab_size {cfg.vocab_size} is below the {base + 256} base tokens")
        words: Counter = Counter()
        chars = 0
        for text in corpus:
            chars += len(text.encode("utf-8"))
            pieces = re.findall(r"\s*\S+|\s+$", text) if cfg.byte_level else [text]
            for p in pieces:
                if p:
                    words[tuple(base + b for b in p.encode("utf-8"))] += 1
        if not words:
            raise TrainerError("empty corpus")
        vocab = {base + b: bytes([b]) for b in range(256)}
        merges: list[MergeRule] = []
        skipped = 0
        unique = len(words)
        from ._merge_learner import MergeLearner
        learner = MergeLearner(words, make=lambda _a, _b, i: base + 256 + i, tie=lambda pair: (-pair[0], -pair[1]))   # ties: the smallest ids win
        while base + 256 + len(merges) < cfg.vocab_size:
            found = learner.best()
            if found is None:
                break
            (a, b), cnt = found
            if cnt < cfg.min_frequency:
                skipped = sum(1 for v in learner.pairs.values() if v < cfg.min_frequency)
                break
            new_id = learner.merge((a, b))
            vocab[new_id] = vocab[a] + vocab[b]
            merges.append(MergeRule(a, b, new_id, cnt))
        special = {t: i for i, t in enumerate(SPECIAL_TOKENS)} if cfg.add_special_tokens else {}
        stats = TrainingStats(base + 256, base + 256 + len(merges), len(merges), skipped, chars, unique)
        return TrainedTokenizer(vocab, merges, special, stats)


# ---- serialisable state -------------------------------------------------------------------------------------------------------
class SerializationError(ValueError):
    pass


def base64_encode(data: bytes) -> str:
    return base64.b64encode(data).decode("ascii")


def base64_decode(text: str) -> bytes:
    try:
        return base64.b64decode(text.encode("ascii"), validate=True)
    except Exception as e:  # noqa: BLE001
        raise SerializationError(f"invalid base64: {e}") from None


@dataclass
class TokenizerState:
    """A snapshot that round-trips through text: token bytes are base64, so any byte sequence survives."""
    vocab: dict[int, bytes] = field(default_factory=dict)
    merges: list[tuple[int, int, int]] = field(default_factory=list)
    special_tokens: dict[str, int] = field(default_factory=dict)

    MAGIC = "oxibonsai-tokenizer-state 1"

    @classmethod
    def from_trained(cls, t: TrainedTokenizer) -> "TokenizerState":
        return cls(dict(t.vocab), [(m.left, m.right, m.merged) for m in t.merges], dict(t.special_tokens))

    def vocab_size(self) -> int:
        return len(self.vocab) + len(self.special_tokens)

    def save(self) -> str:
        lines = [self.MAGIC, f"vocab {len(self.vocab)}"]
        lines += [f"{i} {base64_encode(b)}" for i, b in sorted(self.vocab.items())]
        lines.append(f"merges {len(self.merges)}")
        lines += [f"{a} {b} {m}" for a, b, m in self.merges]
        lines.append(f"special {len(self.special_tokens)}")
        lines += [f"{i} {base64_encode(t.encode('utf-8'))}" for t, i in sorted(self.special_tokens.items(), key=lambda kv: kv[1])]
        return "\n".join(lines) + "\n"

    @classmethod
    def load(cls, text: str) -> "TokenizerState":
        lines = text.splitlines()
        if not lines or lines[0] != cls.MAGIC:
            raise SerializationError("not a tokenizer state (bad header)")
        st, pos = cls(), 1

        def section(name: str) -> int:
            nonlocal pos
            if pos >= len(lines) or not lines[pos].startswith(name + " "):
                raise SerializationError(f"line {pos + 1}: expected '{name} <count>'")
            try:
                n = int(lines[pos].split()[1])
            except (IndexError, ValueError):
                raise SerializationError(f"line {pos + 1}: bad count") from None
            pos += 1
            if pos + n > len(lines):
                raise SerializationError(f"section '{name}' is truncated")
            return n
        try:
            for _ in range(section("vocab")):
                i, b = lines[pos].split(" ", 1)
                st.vocab[int(i)] = base64_decode(b)
                pos += 1
            for _ in range(section("merges")):
                a, b, m = (int(x) for x in lines[pos].split())
                st.merges.append((a, b, m))
                pos += 1
            for _ in range(section("special")):
                i, b = lines[pos].split(" ", 1)
                st.special_tokens[base64_decode(b).decode("utf-8")] = int(i)
                pos += 1
        except SerializationError:
            raise
        except Exception as e:  # noqa: BLE001
            raise SerializationError(f"line {pos + 1}: {e}") from None
        return st

    def save_to(self, path: str) -> None:
        with open(path, "w", encoding="ascii") as f:
            f.write(self.save())

    @classmethod
    def load_from(cls, path: str) -> "TokenizerState":
        with open(path, encoding="ascii") as f:
            return cls.load(f.read())

    def to_tokenizer(self):
        stats = TrainingStats(0, len(self.vocab), len(self.merges), 0, 0, 0)
        merges = [MergeRule(a, b, m, 0) for a, b, m in self.merges]
        return TrainedTokenizer(dict(self.vocab), merges, dict(self.special_tokens), stats).to_tokenizer()


# ---- streaming decoder over token ids -----------------------------------------------------------------------------------------
class IncompleteUtf8(ValueError):
    pass


class TokenStreamDecoder:
    """Feeds token ids, yields text as soon as whole characters are available; bytes of a character that is split over
    tokens wait for the rest."""

    def __init__(self, tokenizer):
        self.tokenizer = tokenizer
        self.reset()

    def reset(self) -> None:
        self._pending = b""
        self._bytes = self._tokens = 0

    def push_token(self, token: int) -> str:
        data = self.tokenizer.token_bytes(token)
        self._tokens += 1
        self._bytes += len(data)
        buf = self._pending + data
        end = len(buf)
        for back in range(1, min(4, end) + 1):
            b = buf[end - back]
            if b & 0xC0 == 0x80:
                continue
            need = 1 if b < 0x80 else 2 if b >> 5 == 0b110 else 3 if b >> 4 == 0b1110 else 4 if b >> 3 == 0b11110 else 1
            if need > back:
                end -= back
            break
        out, self._pending = buf[:end], buf[end:]
        return out.decode("utf-8", errors="replace")

    def push_tokens(self, tokens: Iterable[int]) -> str:
        return "".join(self.push_token(t) for t in tokens)

    def pending_len(self) -> int:
        return len(self._pending)

    def total_bytes(self) -> int:
        return self._bytes

    def total_tokens(self) -> int:
        return self._tokens

    def finish(self) -> str:
        """Ends the stream; bytes that never completed a character are an error (use :meth:`finish_lossy` to keep going)."""
        if self._pending:
            n = len(self._pending)
            self._pending = b""
            raise IncompleteUtf8(f"{n} trailing byte(s) do not form a character")
        return ""

    def finish_lossy(self) -> str:
        out, self._pending = self._pending.decode("utf-8", errors="replace"), b""
        return out

"""RAG, remaining surface: rich chunks and a registry of chunking strategies, a language-aware code chunker, validated
metadata filters, a retriever with configuration, lexical re-ranking and filtered retrieval, retriever snapshots that
carry the embedder's state, and pipeline statistics.

Reference: crates/oxibonsai-rag - advanced_chunker.rs (``RichChunk``, ``ChunkStrategy``, ``SentenceChunker``,
``RecursiveCharSplitter``, ``SlidingWindowChunker``, ``MarkdownChunker``, ``ChunkerRegistry::default_registry``),
code_chunker.rs (``Language::from_extension``; Rust items / Python ``def`` + ``class`` / depth-1 JSON children, plain text
falls back to the recursive splitter), metadata_filter.rs (``validate``, ``eq`` / ``neq`` / ``exists``), distance.rs
(``is_similarity``, ``to_score``), retriever.rs (``RetrieverConfig`` top_k / min_score / rerank; the re-ranker adds 0.02 per
shared query token, at most 0.1, capped at a score of 1), persistence.rs (``IndexSnapshot`` version check,
``RetrieverSnapshot`` save / load), pipeline.rs (``PipelineStats``).
"""
from __future__ import annotations

import json
import math
import re
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Iterable, Sequence

import numpy as np

from . import (Chunk, Distance, IdentityEmbedder, MetadataFilter, SearchHit, TfIdfEmbedder, VectorStore, _tokens, chunk_markdown, chunk_recursive,
               chunk_sentences, chunk_sliding)

SNAPSHOT_VERSION = 1


# ---- rich chunks and strategies -----------------------------------------------------------------------------------------------
@dataclass
class RichChunk:
    text: str
    char_start: int
    char_end: int
    chunk_index: int
    metadata: dict[str, str] = field(default_factory=dict)

    def __len__(self) -> int:
        return len(self.text)

    def is_empty(self) -> bool:
        return not self.text.strip()

    def word_count(self) -> int:
        return len(self.text.split())

    @classmethod
    def of(cls, c: Chunk, strategy: str) -> "RichChunk":
        return cls(c.text, c.start, c.end, c.index, {"strategy": strategy, **{k: str(v) for k, v in c.metadata.items()}})


class ChunkStrategy:
    """A named way of cutting a document; ``chunk`` returns rich chunks with character offsets into the document."""
    name = "strategy"

    def chunk(self, text: str) -> list[RichChunk]:
        raise NotImplementedError


class SentenceChunker(ChunkStrategy):
    name = "sentence"

    def __init__(self, max_chars: int = 512, overlap_sentences: int = 0):
        self.max_chars, self.overlap = max_chars, overlap_sentences

    def with_overlap(self, sentences: int) -> "SentenceChunker":
        self.overlap = sentences
        return self

    def chunk(self, text: str) -> list[RichChunk]:
        if not self.overlap:
            return [RichChunk.of(c, self.name) for c in chunk_sentences(text, self.max_chars)]
        sents = chunk_sentences(text, 1)                      # one sentence per chunk, then packed with a shared tail
        out, i = [], 0
        while i < len(sents):
            j, size = i, 0
            while j < len(sents) and (j == i or size + len(sents[j].text) <= self.max_chars):
                size += len(sents[j].text)
                j += 1
            out.append(RichChunk(text[sents[i].start:sents[j - 1].end], sents[i].start, sents[j - 1].end, len(out), {"strategy": self.name}))
            if j >= len(sents):
                break
            i = max(i + 1, j - self.overlap)
        return out


class RecursiveCharSplitter(ChunkStrategy):
    name = "recursive"

    def __init__(self, max_chars: int = 512):
        self.max_chars, self.separators, self.overlap = max_chars, self.default_separators(), 0

    @staticmethod
    def default_separators() -> tuple[str, ...]:
        return ("\n\n", "\n", ". ", " ", "")

    def with_separators(self, separators: Sequence[str]) -> "RecursiveCharSplitter":
        self.separators = tuple(separators)
        return self

    def with_overlap(self, chars: int) -> "RecursiveCharSplitter":
        self.overlap = chars
        return self

    def chunk(self, text: str) -> list[RichChunk]:
        out = []
        for c in chunk_recursive(text, self.max_chars, self.separators):
            s = max(0, c.start - self.overlap) if out else c.start        # an overlap reaches back into the previous chunk
            out.append(RichChunk(text[s:c.end], s, c.end, len(out), {"strategy": self.name}))
        return out


class SlidingWindowChunker(ChunkStrategy):
    name = "sliding"

    def __init__(self, window: int = 512, stride: int | None = None):
        self.window, self.stride = window, stride or window
        if not 0 < self.stride <= self.window:
            raise ValueError("need 0 < stride <= window")

    @classmethod
    def non_overlapping(cls, window: int) -> "SlidingWindowChunker":
        return cls(window, window)

    @classmethod
    def with_50pct_overlap(cls, window: int) -> "SlidingWindowChunker":
        return cls(window, max(1, window // 2))

    def chunk(self, text: str) -> list[RichChunk]:
        return [RichChunk.of(c, self.name) for c in chunk_sliding(text, self.window, self.stride)]


class MarkdownChunker(ChunkStrategy):
    name = "markdown"

    def __init__(self, max_chars: int = 512):
        self.max_chars = max_chars

    def chunk(self, text: str) -> list[RichChunk]:
        return [RichChunk.of(c, self.name) for c in chunk_markdown(text, self.max_chars)]


class ChunkerRegistry:
    def __init__(self):
        self._by_name: dict[str, ChunkStrategy] = {}

    def register(self, strategy: ChunkStrategy) -> None:
        self._by_name[strategy.name] = strategy

    def chunk(self, name: str, text: str) -> list[RichChunk]:
        if name not in self._by_name:
            raise KeyError(f"unknown chunking strategy {name!r}; available: {', '.join(self.available_strategies())}")
        return self._by_name[name].chunk(text)

    def available_strategies(self) -> list[str]:
        return sorted(self._by_name)

    @classmethod
    def default_registry(cls) -> "ChunkerRegistry":
        r = cls()
        for s in (SentenceChunker(512), RecursiveCharSplitter(512), SlidingWindowChunker.non_overlapping(512), MarkdownChunker(512)):
            r.register(s)
        return r


# ---- code ---------------------------------------------------------------------------------------------------------------------
class Language(Enum):
    RUST = "rust"
    PYTHON = "python"
    JSON = "json"
    PLAIN = "plain"

    @classmethod
    def from_extension(cls, ext: str) -> "Language":
        return {"rs": cls.RUST, "py": cls.PYTHON, "json": cls.JSON}.get(ext.lower().lstrip("."), cls.PLAIN)


_ITEM = {Language.RUST: re.compile(r"^(?:pub(?:\([a-z]+\))?\s+)?(?:async\s+)?(?:fn|impl|struct|enum|mod|trait)\b", re.M),
         Language.PYTHON: re.compile(r"^(?:class|def|async\s+def)\b", re.M)}


class CodeChunker(ChunkStrategy):
    """Cuts source files at top-level items (offsets at the start of a line), JSON at its depth-1 children; pieces below
    ``min_chunk_chars`` are merged into their neighbour, pieces above the window are split recursively."""
    name = "code"

    def __init__(self, language: Language = Language.PLAIN):
        self._language, self.fallback_window, self.min_chunk_chars = language, 512, 16

    def with_fallback_window(self, chars: int) -> "CodeChunker":
        self.fallback_window = chars
        return self

    def with_min_chunk_chars(self, chars: int) -> "CodeChunker":
        self.min_chunk_chars = chars
        return self

    def language(self) -> Language:
        return self._language

    def _fallback(self, text: str, base: int = 0) -> list[tuple[int, int]]:
        return [(base + c.start, base + c.end) for c in chunk_recursive(text, self.fallback_window)]

    def _json_spans(self, text: str) -> list[tuple[int, int]] | None:
        try:
            doc = json.loads(text)
        except json.JSONDecodeError:
            return None
        if not isinstance(doc, (dict, list)) or not doc:
            return None
        # scan for the depth-1 children: between the outer brackets, cut at commas that are at depth 1 and outside strings
        spans, depth, in_str, esc, start = [], 0, False, False, None
        for i, ch in enumerate(text):
            if in_str:
                esc = not esc and ch == "\\"
                if ch == '"' and not esc and text[i - 1] != "\\":
                    in_str = False
                continue
            if ch == '"':
                in_str = True
                if depth == 1 and start is None:
                    start = i
            elif ch in "{[":
                depth += 1
                if depth == 2 and start is None:
                    start = i
            elif ch in "}]":
                if depth == 1 and start is not None:
                    spans.append((start, i))
                    start = None
                depth -= 1
            elif ch == "," and depth == 1:
                if start is not None:
                    spans.append((start, i))
                start = None
            elif depth == 1 and start is None and not ch.isspace():
                start = i
        return [(s, s + len(text[s:e].rstrip())) for s, e in spans if text[s:e].strip()]

    def chunk(self, text: str) -> list[RichChunk]:
        lang = self._language
        spans: list[tuple[int, int]] | None = None
        if lang in _ITEM:
            cuts = sorted({0, len(text), *(m.start() for m in _ITEM[lang].finditer(text))})
            spans = [(a, b) for a, b in zip(cuts, cuts[1:]) if text[a:b].strip()]
        elif lang is Language.JSON:
            spans = self._json_spans(text)
        if not spans:
            spans = self._fallback(text)
        merged: list[tuple[int, int]] = []
        for a, b in spans:                                   # short pieces (a stray import line, a blank header) join what follows
            if merged and merged[-1][1] - merged[-1][0] < self.min_chunk_chars:
                merged[-1] = (merged[-1][0], b)
            else:
                merged.append((a, b))
        if len(merged) > 1 and merged[-1][1] - merged[-1][0] < self.min_chunk_chars:
            last = merged.pop()
            merged[-1] = (merged[-1][0], last[1])
        out: list[RichChunk] = []
        for a, b in merged:
            pieces = [(a, b)] if b - a <= 4 * self.fallback_window else self._fallback(text[a:b], a)
            for s, e in pieces:
                out.append(RichChunk(text[s:e], s, e, len(out), {"strategy": self.name, "language": lang.value}))
        return out


# ---- metadata filters and distances -------------------------------------------------------------------------------------------
_OPS = {"eq", "ne", "in", "gt", "lt", "contains", "exists", "and", "or", "not"}


def validate_filter(f: MetadataFilter, depth: int = 0) -> None:
    """Raises ``ValueError`` for an unknown operator, a missing key, a combinator without children, ``not`` with other than
    one child, ``in`` without a collection, or nesting deeper than 32."""
    if depth > 32:
        raise ValueError("metadata filter is nested deeper than 32 levels")
    if f.op not in _OPS:
        raise ValueError(f"unknown filter operator {f.op!r}")
    if f.op in ("and", "or", "not"):
        if not f.children or (f.op == "not" and len(f.children) != 1):
            raise ValueError(f"'{f.op}' needs {'exactly one child' if f.op == 'not' else 'at least one child'}")
        for c in f.children:
            validate_filter(c, depth + 1)
        return
    if not f.key:
        raise ValueError(f"'{f.op}' needs a key")
    if f.op == "in" and not isinstance(f.value, (list, tuple, set, frozenset)):
        raise ValueError("'in' needs a collection of values")
    if f.op in ("gt", "lt") and not isinstance(f.value, (int, float)):
        raise ValueError(f"'{f.op}' needs a number")


def filter_neq(key: str, value: Any) -> MetadataFilter:
    return MetadataFilter("ne", key, value)


def filter_exists(key: str) -> MetadataFilter:
    return MetadataFilter("exists", key)


def is_similarity(d: Distance) -> bool:
    """Cosine and dot product grow with closeness; Euclidean and Manhattan shrink."""
    return d in (Distance.COSINE, Distance.DOT)


def is_distance(d: Distance) -> bool:
    return not is_similarity(d)


def compute_distance(d: Distance, a: Sequence[float], b: Sequence[float]) -> float:
    """The raw metric value (a distance for Euclidean / Manhattan, a similarity otherwise); mismatched lengths and
    non-finite results raise ``ValueError``."""
    x, y = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    if x.shape != y.shape or x.ndim != 1:
        raise ValueError(f"dimension mismatch: {x.shape} against {y.shape}")
    with np.errstate(over="ignore", invalid="ignore"):
        return _metric(d, x, y)


def _metric(d: Distance, x: np.ndarray, y: np.ndarray) -> float:
    if d is Distance.DOT:
        v = float(x @ y)
    elif d is Distance.COSINE:
        n = float(np.linalg.norm(x) * np.linalg.norm(y))
        v = float(x @ y) / n if n > 0 else 0.0
    elif d is Distance.EUCLIDEAN:
        v = float(np.linalg.norm(x - y))
    else:
        v = float(np.abs(x - y).sum())
    if not math.isfinite(v):
        raise ValueError("non-finite distance")
    return v


def to_score(d: Distance, value: float) -> float:
    """Larger is always better."""
    return value if is_similarity(d) else -value


def store_memory_bytes(store: VectorStore) -> int:
    return store.vectors.nbytes + sum(len(t.encode("utf-8")) for t in store.texts) + sum(len(json.dumps(m)) for m in store.metadata)


def search_with_threshold(store: VectorStore, query: Sequence[float], k: int, threshold: float) -> list[SearchHit]:
    return store.search(query, k, None, threshold)


def clear_store(store: VectorStore) -> None:
    store.clear()


# ---- retriever ----------------------------------------------------------------------------------------------------------------
@dataclass
class RetrieverConfig:
    top_k: int = 4
    min_score: float | None = None
    rerank: bool = False

    def with_top_k(self, k: int) -> "RetrieverConfig":
        self.top_k = k
        return self

    def with_min_score(self, s: float) -> "RetrieverConfig":
        self.min_score = s
        return self

    def with_rerank(self, on: bool = True) -> "RetrieverConfig":
        self.rerank = on
        return self


def rerank(hits: list[SearchHit], query: str) -> list[SearchHit]:
    """Lexical boost on top of the dense score: +0.02 per query token the chunk contains, at most +0.1, score capped at 1."""
    q = set(_tokens(query))
    out = []
    for h in hits:
        overlap = len(q & set(_tokens(h.text)))
        score = min(1.0, h.score + min(0.1, 0.02 * overlap)) if overlap else h.score
        out.append(SearchHit(h.id, score, h.text, h.metadata))
    out.sort(key=lambda h: -h.score)
    return out


class ConfiguredRetriever:
    """Chunks, embeds and stores documents; retrieves with the configured top-k, score floor and optional re-ranking."""

    def __init__(self, embedder=None, config: RetrieverConfig | None = None, distance: Distance = Distance.COSINE,
                 chunker: Callable[[str], list] | None = None, store: VectorStore | None = None):
        self.embedder = embedder or IdentityEmbedder()
        self.config = config or RetrieverConfig()
        self._store = store or VectorStore(self.embedder.dim, distance)
        self._chunker = chunker or (lambda text: RecursiveCharSplitter(512).chunk(text))
        self.documents = 0

    @classmethod
    def from_parts(cls, embedder, store: VectorStore, config: RetrieverConfig | None = None, documents: int = 0) -> "ConfiguredRetriever":
        r = cls(embedder, config, store.distance, store=store)
        r.documents = documents
        return r

    def add_document(self, text: str, metadata: dict | None = None) -> int:
        n = 0
        for c in self._chunker(text):
            if not c.text.strip():
                continue
            self._store.add(self.embedder.embed(c.text), c.text, {**(metadata or {}), "doc": self.documents, "chunk": n})
            n += 1
        self.documents += 1
        return n

    def add_documents(self, texts: Iterable[str]) -> int:
        return sum(self.add_document(t) for t in texts)

    def retrieve(self, query: str, k: int | None = None) -> list[SearchHit]:
        return self.retrieve_filtered(query, None, k)

    def retrieve_filtered(self, query: str, flt: MetadataFilter | None, k: int | None = None) -> list[SearchHit]:
        if flt is not None:
            validate_filter(flt)
        k = k or self.config.top_k
        # re-ranking may promote a hit from just below the cut, so a few more candidates are fetched
        hits = self._store.search(self.embedder.embed(query), k * 3 if self.config.rerank else k, flt, self.config.min_score)
        return (rerank(hits, query) if self.config.rerank else hits)[:k]

    def retrieve_text(self, query: str, k: int | None = None) -> list[str]:
        return [h.text for h in self.retrieve(query, k)]

    def document_count(self) -> int:
        return self.documents

    def chunk_count(self) -> int:
        return len(self._store)

    def store(self) -> VectorStore:
        return self._store


# ---- snapshots ----------------------------------------------------------------------------------------------------------------
def check_version(doc: dict) -> None:
    v = doc.get("version")
    if v != SNAPSHOT_VERSION:
        raise ValueError(f"unsupported snapshot version {v!r} (this build reads version {SNAPSHOT_VERSION})")


def _embedder_state(e) -> dict:
    if isinstance(e, TfIdfEmbedder):
        return {"kind": "tfidf", "dim": e.dim, "n_docs": e.n_docs, "df": e.df}
    if isinstance(e, IdentityEmbedder):
        return {"kind": "identity", "dim": e.dim}
    raise ValueError(f"embedder {type(e).__name__} cannot be snapshotted; save the store and rebuild the embedder yourself")


def _embedder_from(state: dict):
    if state["kind"] == "tfidf":
        e = TfIdfEmbedder(state["dim"])
        e.n_docs, e.df = int(state["n_docs"]), {k: int(v) for k, v in state["df"].items()}
        return e
    if state["kind"] == "identity":
        return IdentityEmbedder(state["dim"])
    raise ValueError(f"unknown embedder kind {state['kind']!r}")


@dataclass
class RetrieverSnapshot:
    """Everything needed to answer the same queries after a restart: store, embedder state, configuration, counters."""
    doc: dict

    @classmethod
    def to_snapshot(cls, r: ConfiguredRetriever) -> "RetrieverSnapshot":
        return cls({"version": SNAPSHOT_VERSION, "index": json.loads(r.store().to_json()), "embedder": _embedder_state(r.embedder),
                    "config": {"top_k": r.config.top_k, "min_score": r.config.min_score, "rerank": r.config.rerank}, "documents": r.documents})

    def from_snapshot(self) -> ConfiguredRetriever:
        check_version(self.doc)
        store = VectorStore.from_json(json.dumps(self.doc["index"]))
        return ConfiguredRetriever.from_parts(_embedder_from(self.doc["embedder"]), store, RetrieverConfig(**self.doc["config"]), int(self.doc["documents"]))

    def save_json(self) -> str:
        return json.dumps(self.doc)

    @classmethod
    def load_json(cls, text: str) -> "RetrieverSnapshot":
        doc = json.loads(text)
        check_version(doc)
        return cls(doc)

    def save(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as f:
            f.write(self.save_json())

    @classmethod
    def load(cls, path: str) -> "RetrieverSnapshot":
        with open(path, encoding="utf-8") as f:
            return cls.load_json(f.read())


# ---- pipeline statistics ------------------------------------------------------------------------------------------------------
@dataclass
class PipelineStats:
    documents_indexed: int
    chunks_indexed: int
    embedding_dim: int
    store_memory_bytes: int


def pipeline_stats(pipeline) -> PipelineStats:
    """Statistics of a :class:`~oxibonsai_b200.rag.RagPipeline` or a :class:`ConfiguredRetriever`."""
    store = pipeline.store() if callable(getattr(pipeline, "store", None)) else pipeline.store
    return PipelineStats(int(pipeline.documents), len(store), store.dim, store_memory_bytes(store))

"""Retrieval-augmented generation: chunkers, embedders, vector store with metadata filters, retriever, pipeline,
JSON snapshots.

Reference: crates/oxibonsai-rag (chunkers: char / sentence / paragraph / markdown / recursive / sliding / code / semantic;
``Embedder`` trait with ``IdentityEmbedder`` and ``TfIdfEmbedder`` in embedding.rs:19-123; flat ``VectorStore`` with
``Distance`` metrics and ``MetadataFilter`` in vector_store.rs:76-109, distance.rs:31, metadata_filter.rs:52-115;
``Retriever`` in retriever.rs:27-78; ``RagPipeline::index_document`` / ``build_prompt`` in pipeline.rs:23-126; JSON
snapshots in persistence.rs:77-115).  Similarity search over the whole store is one matrix product; with torch and a
GPU available the store can keep its matrix on the device.
"""
from __future__ import annotations

import hashlib
import json
import math
import re
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Iterable, Protocol, Sequence

import numpy as np


# ---- chunkers ---------------------------------------------------------------------------------------------------------------
@dataclass
class Chunk:
    text: str
    start: int
    end: int
    index: int = 0
    metadata: dict = field(default_factory=dict)


def _mk(text: str, spans: Iterable[tuple[int, int]]) -> list[Chunk]:
    out = []
    for s, e in spans:
        if text[s:e].strip():
            out.append(Chunk(text[s:e], s, e, len(out)))
    return out


def chunk_chars(text: str, size: int = 512, overlap: int = 0) -> list[Chunk]:
    if size <= 0 or overlap >= size:
        raise ValueError("need size > overlap >= 0")
    step = size - overlap
    return _mk(text, ((i, min(len(text), i + size)) for i in range(0, max(len(text), 1), step) if i < len(text)))


def chunk_sliding(text: str, window: int = 512, stride: int = 256) -> list[Chunk]:
    return chunk_chars(text, window, window - stride)


_SENT = re.compile(r"[^.!?\n]+[.!?]*\s*|\n+")


def chunk_sentences(text: str, max_chars: int = 512) -> list[Chunk]:
    """Whole sentences packed greedily up to ``max_chars``."""
    spans, cur_s, cur_e = [], None, None
    for m in _SENT.finditer(text):
        s, e = m.span()
        if cur_s is None:
            cur_s, cur_e = s, e
        elif e - cur_s <= max_chars:
            cur_e = e
        else:
            spans.append((cur_s, cur_e))
            cur_s, cur_e = s, e
    if cur_s is not None:
        spans.append((cur_s, cur_e))
    return _mk(text, spans)


def chunk_paragraphs(text: str, max_chars: int = 2000) -> list[Chunk]:
    spans, pos = [], 0
    for m in re.finditer(r"\n\s*\n", text + "\n\n"):
        s, e = pos, m.start()
        pos = m.end()
        while e - s > max_chars:
            spans.append((s, s + max_chars))
            s += max_chars
        if e > s:
            spans.append((s, min(e, len(text))))
    return _mk(text, spans)


def chunk_markdown(text: str, max_chars: int = 2000) -> list[Chunk]:
    """Sections split at headings; each chunk remembers its heading path."""
    heads = [(m.start(), len(m.group(1)), m.group(2).strip()) for m in re.finditer(r"^(#{1,6})\s+(.*)$", text, re.M)]
    bounds = [h[0] for h in heads] + [len(text)]
    if not heads or heads[0][0] > 0:
        bounds = [0] + bounds
        heads = [(0, 0, "")] + heads
    out, path = [], []
    for (pos, level, title), end in zip(heads, bounds[1:]):
        if level:
            path = path[: level - 1] + [title]
        for c in chunk_paragraphs(text[pos:end], max_chars) if end - pos > max_chars else _mk(text, [(pos, end)]):
            s, e = (c.start + pos, c.end + pos) if end - pos > max_chars else (c.start, c.end)
            out.append(Chunk(text[s:e], s, e, len(out), {"heading_path": " > ".join(p for p in path if p)}))
    return out


def chunk_recursive(text: str, max_chars: int = 512, separators: Sequence[str] = ("\n\n", "\n", ". ", " ", "")) -> list[Chunk]:
    """Split on the coarsest separator that yields pieces within ``max_chars``, recursing into oversized pieces."""
    def rec(s: int, e: int, level: int) -> list[tuple[int, int]]:
        if e - s <= max_chars:
            return [(s, e)]
        if level >= len(separators) or separators[level] == "":
            return [(i, min(e, i + max_chars)) for i in range(s, e, max_chars)]
        sep, parts, pos = separators[level], [], s
        while True:
            j = text.find(sep, pos, e)
            if j < 0:
                parts.append((pos, e))
                break
            parts.append((pos, j + len(sep)))
            pos = j + len(sep)
        merged, cs, ce = [], None, None
        for ps, pe in parts:
            if cs is None:
                cs, ce = ps, pe
            elif pe - cs <= max_chars:
                ce = pe
            else:
                merged.append((cs, ce))
                cs, ce = ps, pe
        if cs is not None:
            merged.append((cs, ce))
        return [x for ms, me in merged for x in rec(ms, me, level + 1)]
    return _mk(text, rec(0, len(text), 0))


def chunk_code(text: str, max_chars: int = 1500) -> list[Chunk]:
    """Split before top-level definitions (``def``, ``class``, ``fn``, ``function`` ...), then recursively if too long."""
    starts = [m.start() for m in re.finditer(r"^(?:async\s+def|def|class|fn|pub\s+fn|impl|struct|function|func)\b", text, re.M)]
    bounds = sorted(set([0] + starts + [len(text)]))
    out = []
    for s, e in zip(bounds, bounds[1:]):
        for c in chunk_recursive(text[s:e], max_chars, ("\n\n", "\n", " ", "")):
            out.append(Chunk(c.text, s + c.start, s + c.end, len(out)))
    return out


def chunk_semantic(text: str, embed: Callable[[str], Sequence[float]], threshold: float = 0.5, max_chars: int = 1500) -> list[Chunk]:
    """Sentences are merged while consecutive sentences stay similar; a similarity drop starts a new chunk."""
    sents = chunk_sentences(text, 1)
    if not sents:
        return []
    vecs = [np.asarray(embed(s.text), dtype=np.float64) for s in sents]
    spans, cs, ce = [], sents[0].start, sents[0].end
    for prev, cur, a, b in zip(sents, sents[1:], vecs, vecs[1:]):
        na, nb = np.linalg.norm(a), np.linalg.norm(b)
        sim = float(a @ b / (na * nb)) if na > 0 and nb > 0 else 0.0
        if sim < threshold or cur.end - cs > max_chars:
            spans.append((cs, ce))
            cs = cur.start
        ce = cur.end
    spans.append((cs, ce))
    return _mk(text, spans)


# ---- embedders ----------------------------------------------------------------------------------------------------------------
class Embedder(Protocol):
    dim: int

    def embed(self, text: str) -> np.ndarray: ...


def _tokens(text: str) -> list[str]:
    return re.findall(r"[\w']+", text.lower())


def _bucket(tok: str, dim: int) -> tuple[int, float]:
    h = int.from_bytes(hashlib.blake2b(tok.encode(), digest_size=8).digest(), "little")
    return h % dim, (1.0 if (h >> 63) & 1 == 0 else -1.0)


class IdentityEmbedder:
    """Hashed bag of words (signed feature hashing), L2-normalised."""

    def __init__(self, dim: int = 512):
        self.dim = dim

    def embed(self, text: str) -> np.ndarray:
        v = np.zeros(self.dim, dtype=np.float32)
        for t in _tokens(text):
            i, s = _bucket(t, self.dim)
            v[i] += s
        n = float(np.linalg.norm(v))
        return v / n if n > 0 else v


class TfIdfEmbedder:
    """Feature-hashed TF-IDF; ``fit`` learns document frequencies."""

    def __init__(self, dim: int = 512):
        self.dim, self.n_docs = dim, 0
        self.df: dict[str, int] = {}

    def fit(self, docs: Iterable[str]) -> "TfIdfEmbedder":
        for d in docs:
            self.n_docs += 1
            for t in set(_tokens(d)):
                self.df[t] = self.df.get(t, 0) + 1
        return self

    def idf(self, tok: str) -> float:
        return math.log((1 + self.n_docs) / (1 + self.df.get(tok, 0))) + 1.0

    def embed(self, text: str) -> np.ndarray:
        v = np.zeros(self.dim, dtype=np.float32)
        toks = _tokens(text)
        for t in toks:
            i, s = _bucket(t, self.dim)
            v[i] += s * self.idf(t) / max(1, len(toks))
        n = float(np.linalg.norm(v))
        return v / n if n > 0 else v


# ---- vector store -------------------------------------------------------------------------------------------------------------------
class Distance(Enum):
    COSINE = "cosine"
    DOT = "dot"
    EUCLIDEAN = "euclidean"
    MANHATTAN = "manhattan"

    def scores(self, matrix: np.ndarray, q: np.ndarray) -> np.ndarray:
        """Higher = closer, for every metric."""
        if self == Distance.DOT:
            return matrix @ q
        if self == Distance.COSINE:
            n = np.linalg.norm(matrix, axis=1) * (np.linalg.norm(q) or 1.0)
            return (matrix @ q) / np.where(n > 0, n, 1.0)
        # the difference matrix is formed a cache-sized block of rows at a time (the whole of it is 100 MB at 100k x 256)
        out = np.empty(len(matrix), dtype=np.float32)
        step = max(1, (1 << 19) // max(1, matrix.shape[1]))
        for a in range(0, len(matrix), step):
            d = matrix[a:a + step] - q[None, :]
            out[a:a + step] = -np.sqrt(np.einsum("ij,ij->i", d, d)) if self == Distance.EUCLIDEAN else -np.abs(d).sum(1)
        return out


@dataclass
class MetadataFilter:
    """``op``: eq | ne | in | gt | lt | contains | exists | and | or | not."""
    op: str
    key: str = ""
    value: Any = None
    children: list["MetadataFilter"] = field(default_factory=list)

    def matches(self, md: dict) -> bool:
        if self.op == "and":
            return all(c.matches(md) for c in self.children)
        if self.op == "or":
            return any(c.matches(md) for c in self.children)
        if self.op == "not":
            return not self.children[0].matches(md)
        if self.op == "exists":
            return self.key in md
        if self.key not in md:
            return False
        v = md[self.key]
        return {"eq": lambda: v == self.value, "ne": lambda: v != self.value, "in": lambda: v in self.value, "gt": lambda: v > self.value,
                "lt": lambda: v < self.value, "contains": lambda: self.value in v}[self.op]()

    @classmethod
    def eq(cls, key, value):
        return cls("eq", key, value)

    @classmethod
    def all_of(cls, *fs):
        return cls("and", children=list(fs))

    @classmethod
    def any_of(cls, *fs):
        return cls("or", children=list(fs))


@dataclass
class SearchHit:
    id: int
    score: float
    text: str
    metadata: dict


class VectorStore:
    """Flat store: the vectors sit in one matrix that grows geometrically, with their norms beside them, so that indexing
    and querying in turns costs no re-packing and a query is one matrix-vector product plus a partial sort."""

    def __init__(self, dim: int, distance: Distance = Distance.COSINE):
        self.dim, self.distance = dim, distance
        self._buf = np.empty((0, dim), dtype=np.float32)
        self._norms = np.empty(0, dtype=np.float32)
        self._n = 0
        self.texts: list[str] = []
        self.metadata: list[dict] = []

    @property
    def vectors(self) -> np.ndarray:
        """The stored vectors as one [n, dim] view."""
        return self._buf[:self._n]

    def add(self, vector: Sequence[float], text: str, metadata: dict | None = None) -> int:
        v = np.asarray(vector, dtype=np.float32)
        if v.shape != (self.dim,):
            raise ValueError(f"expected dimension {self.dim}, got {v.shape}")
        if self._n == len(self._buf):
            cap = max(64, 2 * len(self._buf))
            self._buf = np.concatenate([self._buf, np.empty((cap - self._n, self.dim), dtype=np.float32)])
            self._norms = np.concatenate([self._norms, np.empty(cap - self._n, dtype=np.float32)])
        self._buf[self._n] = v
        self._norms[self._n] = np.linalg.norm(v)
        self._n += 1
        self.texts.append(text)
        self.metadata.append(dict(metadata or {}))
        return self._n - 1

    def __len__(self) -> int:
        return self._n

    def clear(self) -> None:
        self._buf, self._norms, self._n = np.empty((0, self.dim), dtype=np.float32), np.empty(0, dtype=np.float32), 0
        self.texts.clear()
        self.metadata.clear()

    def _scores(self, q: np.ndarray) -> np.ndarray:
        m = self.vectors
        if self.distance == Distance.COSINE:                       # the stored norms save a pass over the matrix
            n = self._norms[:self._n] * (np.linalg.norm(q) or 1.0)
            return (m @ q) / np.where(n > 0, n, 1.0)
        return self.distance.scores(m, q)

    def search(self, query: Sequence[float], k: int = 4, flt: MetadataFilter | None = None, min_score: float | None = None) -> list[SearchHit]:
        if self._n == 0 or k <= 0:
            return []
        s = self._scores(np.asarray(query, dtype=np.float32))
        # without a filter only the k best are ever looked at: select them first, sort those (ties by index, as a stable
        # sort of the whole row would give them)
        want = min(self._n, k if flt is None else self._n)
        if want < self._n:
            cut = np.partition(s, self._n - want)[self._n - want]
            cand = np.flatnonzero(s >= cut)
        else:
            cand = np.arange(self._n)
        order = cand[np.argsort(-s[cand], kind="stable")]
        out = []
        for i in order:
            if flt is not None and not flt.matches(self.metadata[i]):
                continue
            if min_score is not None and s[i] < min_score:
                break
            out.append(SearchHit(int(i), float(s[i]), self.texts[i], self.metadata[i]))
            if len(out) == k:
                break
        return out

    def remove(self, idx: int) -> None:
        if not -self._n <= idx < self._n:
            raise IndexError(idx)
        idx %= self._n
        self._buf[idx:self._n - 1] = self._buf[idx + 1:self._n]
        self._norms[idx:self._n - 1] = self._norms[idx + 1:self._n]
        self._n -= 1
        del self.texts[idx], self.metadata[idx]

    # JSON snapshots
    def to_json(self) -> str:
        return json.dumps({"version": 1, "dim": self.dim, "distance": self.distance.value, "entries": [
            {"vector": [float(x) for x in v], "text": t, "metadata": m} for v, t, m in zip(self.vectors, self.texts, self.metadata)]})

    @classmethod
    def from_json(cls, data: str) -> "VectorStore":
        j = json.loads(data)
        if j.get("version") != 1:
            raise ValueError("unsupported snapshot version")
        s = cls(j["dim"], Distance(j["distance"]))
        for e in j["entries"]:
            s.add(e["vector"], e["text"], e["metadata"])
        return s

    def save(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as f:
            f.write(self.to_json())

    @classmethod
    def load(cls, path: str) -> "VectorStore":
        with open(path, encoding="utf-8") as f:
            return cls.from_json(f.read())


class Retriever:
    def __init__(self, store: VectorStore, embedder, top_k: int = 4, min_score: float | None = None):
        self.store, self.embedder, self.top_k, self.min_score = store, embedder, top_k, min_score

    def retrieve(self, query: str, k: int | None = None, flt: MetadataFilter | None = None) -> list[SearchHit]:
        return self.store.search(self.embedder.embed(query), k or self.top_k, flt, self.min_score)


@dataclass
class RagConfig:
    chunker: str = "recursive"
    chunk_chars: int = 512
    top_k: int = 4
    max_context_chars: int = 4000
    template: str = "Use the following context to answer the question.\n\n{context}\n\nQuestion: {question}\nAnswer:"


class RagPipeline:
    def __init__(self, embedder=None, config: RagConfig | None = None, distance: Distance = Distance.COSINE):
        self.config = config or RagConfig()
        self.embedder = embedder or IdentityEmbedder()
        self.store = VectorStore(self.embedder.dim, distance)
        self.retriever = Retriever(self.store, self.embedder, self.config.top_k)
        self.documents = 0

    def _chunks(self, text: str) -> list[Chunk]:
        c, n = self.config.chunker, self.config.chunk_chars
        table = {"char": lambda: chunk_chars(text, n), "sentence": lambda: chunk_sentences(text, n), "paragraph": lambda: chunk_paragraphs(text, n),
                 "markdown": lambda: chunk_markdown(text, n), "recursive": lambda: chunk_recursive(text, n), "sliding": lambda: chunk_sliding(text, n, max(1, n // 2)),
                 "code": lambda: chunk_code(text, n), "semantic": lambda: chunk_semantic(text, self.embedder.embed, max_chars=n)}
        if c not in table:
            raise ValueError(f"unknown chunker {c!r}")
        return table[c]()

    def index_document(self, text: str, metadata: dict | None = None) -> int:
        chunks = self._chunks(text)
        for ch in chunks:
            self.store.add(self.embedder.embed(ch.text), ch.text, {**(metadata or {}), **ch.metadata, "doc": self.documents, "chunk": ch.index, "start": ch.start})
        self.documents += 1
        return len(chunks)

    def query(self, question: str, k: int | None = None, flt: MetadataFilter | None = None) -> list[SearchHit]:
        return self.retriever.retrieve(question, k, flt)

    def build_prompt(self, question: str, k: int | None = None, flt: MetadataFilter | None = None) -> str:
        parts, used = [], 0
        for i, h in enumerate(self.query(question, k, flt)):
            if used + len(h.text) > self.config.max_context_chars:
                break
            parts.append(f"[{i + 1}] {h.text.strip()}")
            used += len(h.text)
        return self.config.template.format(context="\n\n".join(parts), question=question)

    def stats(self) -> dict:
        return {"documents": self.documents, "chunks": len(self.store), "dim": self.store.dim, "distance": self.store.distance.value}

"""Serving-side caches and registries: hot reload bookkeeping, multi-model registry / router with LoRA adapter stacks,
LRU model cache with warm-up, exact and semantic response caches, and a navigable-small-world vector index.

Reference: crates/oxibonsai-runtime/src/hot_reload.rs:47-260, multi_model.rs, model_cache.rs, dedup.rs, semantic_cache.rs
and embedding_index.rs (``NswIndex`` / ``EmbeddingIndex``).
"""
from __future__ import annotations

import hashlib
import heapq
import threading
import time
from collections import OrderedDict, deque
from dataclasses import dataclass, field
from typing import Any, Callable, Generic, Sequence, TypeVar

import numpy as np

T = TypeVar("T")


# ---- hot reload -------------------------------------------------------------------------------------------------------------
@dataclass
class ModelVersion:
    generation: int
    path: str
    loaded_at: float = field(default_factory=time.time)
    checksum: str = ""

    def age_seconds(self) -> float:
        return time.time() - self.loaded_at


@dataclass
class ReloadEvent:
    timestamp: float
    generation: int
    path: str
    success: bool
    message: str = ""


class ReloadLog:
    def __init__(self, capacity: int = 256):
        self._events: deque[ReloadEvent] = deque(maxlen=capacity)
        self._total = 0

    def record(self, event: ReloadEvent) -> None:
        self._events.append(event)
        self._total += 1

    def recent_events(self, n: int = 10) -> list[ReloadEvent]:
        return list(self._events)[-n:]

    def total_events(self) -> int:
        return self._total

    def summary(self) -> str:
        ok = sum(e.success for e in self._events)
        return f"{self._total} reloads ({ok} ok, {len(self._events) - ok} failed in the retained window)"


class HotReloadCoordinator:
    """Generation counter + version history; readers compare generations to notice a swap."""

    def __init__(self, max_history: int = 16):
        self._lock = threading.Lock()
        self._history: deque[ModelVersion] = deque(maxlen=max_history)
        self._generation = 0
        self.log = ReloadLog()

    def with_max_history(self, n: int) -> "HotReloadCoordinator":
        self._history = deque(self._history, maxlen=n)
        return self

    def record_reload(self, path: str, checksum: str = "") -> ModelVersion:
        with self._lock:
            self._generation += 1
            v = ModelVersion(self._generation, path, checksum=checksum)
            self._history.append(v)
            self.log.record(ReloadEvent(time.time(), v.generation, path, True))
            return v

    def record_failure(self, path: str, message: str) -> None:
        self.log.record(ReloadEvent(time.time(), self._generation, path, False, message))

    def current_generation(self) -> int:
        return self._generation

    def version_history(self) -> list[ModelVersion]:
        return list(self._history)

    def current_version(self) -> ModelVersion | None:
        return self._history[-1] if self._history else None

    def reload_count(self) -> int:
        return self._generation

    def reload(self, path: str, loader: Callable[[str], Any]) -> Any:
        """Loads a new model with ``loader`` and bumps the generation only when loading succeeds."""
        try:
            model = loader(path)
        except Exception as e:
            self.record_failure(path, str(e))
            raise
        self.record_reload(path)
        return model


# ---- multi-model registry ---------------------------------------------------------------------------------------------------------
class ModelId(str):
    """``base`` or ``base:adapter``."""

    def is_base(self) -> bool:
        return ":" not in self

    def base_name(self) -> str:
        return self.split(":", 1)[0]

    def adapter_name(self) -> str | None:
        return self.split(":", 1)[1] if ":" in self else None


@dataclass
class ModelEndpoint:
    model_id: ModelId
    path: str
    adapter: str | None = None
    description: str = ""
    context_length: int = 4096
    status: str = "ready"          # ready | loading | draining | offline
    is_default: bool = False

    def is_available(self) -> bool:
        return self.status == "ready"


class RoutingError(LookupError):
    pass


class ModelRegistry:
    def __init__(self):
        self._endpoints: dict[str, ModelEndpoint] = {}
        self._aliases: dict[str, str] = {}

    def register(self, ep: ModelEndpoint) -> None:
        if ep.is_default:
            for e in self._endpoints.values():
                e.is_default = False
        self._endpoints[str(ep.model_id)] = ep

    def unregister(self, model_id: str) -> bool:
        self._aliases = {a: t for a, t in self._aliases.items() if t != model_id}
        return self._endpoints.pop(model_id, None) is not None

    def add_alias(self, alias: str, model_id: str) -> None:
        if model_id not in self._endpoints:
            raise RoutingError(f"unknown model {model_id!r}")
        self._aliases[alias] = model_id

    def resolve(self, name: str) -> ModelEndpoint | None:
        return self._endpoints.get(self._aliases.get(name, name))

    def default_endpoint(self) -> ModelEndpoint | None:
        return next((e for e in self._endpoints.values() if e.is_default), next(iter(self._endpoints.values()), None))

    def available_endpoints(self) -> list[ModelEndpoint]:
        return [e for e in self._endpoints.values() if e.is_available()]

    def all_endpoints(self) -> list[ModelEndpoint]:
        return list(self._endpoints.values())

    def set_status(self, model_id: str, status: str) -> None:
        self._endpoints[model_id].status = status

    def __len__(self) -> int:
        return len(self._endpoints)


class ModelRouter:
    def __init__(self, registry: ModelRegistry | None = None):
        self.registry = registry or ModelRegistry()

    def route(self, requested: str | None) -> ModelEndpoint:
        ep = self.registry.resolve(requested) if requested else self.registry.default_endpoint()
        if ep is None:
            raise RoutingError(f"no model named {requested!r}")
        if not ep.is_available():
            raise RoutingError(f"model {ep.model_id!r} is {ep.status}")
        return ep

    def route_for_context(self, n_tokens: int) -> ModelEndpoint:
        fits = sorted((e for e in self.registry.available_endpoints() if e.context_length >= n_tokens), key=lambda e: e.context_length)
        if not fits:
            raise RoutingError(f"no available model has a context of {n_tokens} tokens")
        return fits[0]

    def models_list(self) -> list[dict]:
        return [{"id": str(e.model_id), "object": "model", "owned_by": "oxibonsai", "description": e.description, "context_length": e.context_length,
                 "status": e.status} for e in self.registry.all_endpoints()]


@dataclass
class AdapterRef:
    name: str
    weight: float = 1.0


class AdapterStack:
    """Weighted set of LoRA adapters applied together."""

    def __init__(self):
        self.adapters: list[AdapterRef] = []

    def add(self, name: str, weight: float = 1.0) -> "AdapterStack":
        self.adapters.append(AdapterRef(name, weight))
        return self

    def __len__(self) -> int:
        return len(self.adapters)

    def total_weight(self) -> float:
        return sum(a.weight for a in self.adapters)

    def normalize_weights(self) -> None:
        t = self.total_weight()
        if t > 0:
            for a in self.adapters:
                a.weight /= t


# ---- model cache + warm-up ----------------------------------------------------------------------------------------------------------
@dataclass
class ModelEntry:
    model: Any
    memory_bytes: int
    created: float = field(default_factory=time.monotonic)
    last_used: float = field(default_factory=time.monotonic)
    hits: int = 0

    def age(self) -> float:
        return time.monotonic() - self.created

    def idle_time(self) -> float:
        return time.monotonic() - self.last_used

    def is_stale(self, max_idle: float) -> bool:
        return self.idle_time() > max_idle


@dataclass
class ModelCacheConfig:
    max_models: int = 4
    max_memory_bytes: int = 160 << 30      # a B200 holds 180 GB
    max_idle_seconds: float = 3600.0


class ModelCache:
    """LRU cache of loaded engines bounded by count and memory."""

    def __init__(self, config: ModelCacheConfig | None = None):
        self.config = config or ModelCacheConfig()
        self._entries: OrderedDict[str, ModelEntry] = OrderedDict()
        self._lock = threading.Lock()
        self.hits = self.misses = self.evictions = 0

    def get_or_insert(self, key: str, loader: Callable[[], tuple[Any, int]]) -> Any:
        with self._lock:
            e = self._entries.get(key)
            if e is not None:
                e.last_used, e.hits = time.monotonic(), e.hits + 1
                self._entries.move_to_end(key)
                self.hits += 1
                return e.model
            self.misses += 1
        model, nbytes = loader()
        with self._lock:
            self._entries[key] = ModelEntry(model, nbytes)
            while len(self._entries) > self.config.max_models or (self.total_memory_bytes() > self.config.max_memory_bytes and len(self._entries) > 1):
                self._entries.popitem(last=False)
                self.evictions += 1
        return model

    def contains(self, key: str) -> bool:
        return key in self._entries

    def evict(self, key: str) -> bool:
        with self._lock:
            if self._entries.pop(key, None) is not None:
                self.evictions += 1
                return True
            return False

    def evict_stale(self) -> int:
        with self._lock:
            stale = [k for k, e in self._entries.items() if e.is_stale(self.config.max_idle_seconds)]
            for k in stale:
                del self._entries[k]
            self.evictions += len(stale)
            return len(stale)

    def __len__(self) -> int:
        return len(self._entries)

    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0

    def total_memory_bytes(self) -> int:
        return sum(e.memory_bytes for e in self._entries.values())

    def stats(self) -> dict:
        return {"models": len(self), "hits": self.hits, "misses": self.misses, "evictions": self.evictions, "memory_bytes": self.total_memory_bytes()}


class ModelWarmup:
    """Runs a short generation so kernels are loaded and graphs captured before the first request."""

    def __init__(self, tokens: int = 4, prompt: Sequence[int] = (0,) * 17):
        self.tokens, self.prompt, self.done = tokens, list(prompt), False

    def with_tokens(self, n: int) -> "ModelWarmup":
        self.tokens = n
        return self

    def with_prompt(self, prompt: Sequence[int]) -> "ModelWarmup":
        self.prompt = list(prompt)
        return self

    def needs_warmup(self) -> bool:
        return not self.done

    def run(self, generate: Callable[[list[int], int], Any]) -> float:
        t0 = time.perf_counter()
        generate(self.prompt, self.tokens)
        self.done = True
        return time.perf_counter() - t0


# ---- exact response cache ------------------------------------------------------------------------------------------------------------
def request_key(text_or_messages: str | Sequence[dict], **params) -> str:
    h = hashlib.blake2b(digest_size=16)
    if isinstance(text_or_messages, str):
        h.update(text_or_messages.encode())
    else:
        for m in text_or_messages:
            h.update(f"{m.get('role')}\x1f{m.get('content')}\x1e".encode())
    for k in sorted(params):
        h.update(f"{k}={params[k]}".encode())
    return h.hexdigest()


@dataclass
class CachedResponse:
    text: str
    created: float = field(default_factory=time.monotonic)
    ttl: float | None = None
    hits: int = 0

    def is_expired(self) -> bool:
        return self.ttl is not None and time.monotonic() - self.created > self.ttl

    def age(self) -> float:
        return time.monotonic() - self.created


class DedupCache:
    """Identical deterministic requests are answered from memory."""

    def __init__(self, capacity: int = 1024, default_ttl: float | None = 300.0):
        self.capacity, self.default_ttl = capacity, default_ttl
        self._d: OrderedDict[str, CachedResponse] = OrderedDict()
        self.hits = self.misses = 0
        self._lock = threading.Lock()

    def get(self, key: str) -> str | None:
        with self._lock:
            e = self._d.get(key)
            if e is None or e.is_expired():
                if e is not None:
                    del self._d[key]
                self.misses += 1
                return None
            e.hits += 1
            self.hits += 1
            self._d.move_to_end(key)
            return e.text

    def insert(self, key: str, text: str, ttl: float | None = ...) -> None:
        with self._lock:
            self._d[key] = CachedResponse(text, ttl=self.default_ttl if ttl is ... else ttl)
            self._d.move_to_end(key)
            while len(self._d) > self.capacity:
                self._d.popitem(last=False)

    def evict_expired(self) -> int:
        with self._lock:
            dead = [k for k, e in self._d.items() if e.is_expired()]
            for k in dead:
                del self._d[k]
            return len(dead)

    def __len__(self) -> int:
        return len(self._d)

    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0

    def stats(self) -> dict:
        return {"entries": len(self), "hits": self.hits, "misses": self.misses, "hit_rate": self.hit_rate()}

    def clear(self) -> None:
        self._d.clear()


# ---- NSW index + semantic cache ---------------------------------------------------------------------------------------------------------
@dataclass
class NswConfig:
    max_neighbors: int = 16
    ef_construction: int = 64
    ef_search: int = 32


@dataclass
class NswSearchResult:
    index: int
    distance: float


class NswIndex:
    """Single-layer navigable small world graph under cosine distance."""

    def __init__(self, dim: int, config: NswConfig | None = None):
        self.dim, self.config = dim, config or NswConfig()
        self.vectors: list[np.ndarray] = []
        self.neighbors: list[list[int]] = []

    def __len__(self) -> int:
        return len(self.vectors)

    def _dist(self, a: np.ndarray, i: int) -> float:
        return 1.0 - float(np.dot(a, self.vectors[i]))

    def _search(self, q: np.ndarray, ef: int) -> list[tuple[float, int]]:
        if not self.vectors:
            return []
        entry = 0
        d0 = self._dist(q, entry)
        cand, best, seen = [(d0, entry)], [(-d0, entry)], {entry}
        while cand:
            d, i = heapq.heappop(cand)
            if d > -best[0][0] and len(best) >= ef:
                break
            for j in self.neighbors[i]:
                if j in seen:
                    continue
                seen.add(j)
                dj = self._dist(q, j)
                if len(best) < ef or dj < -best[0][0]:
                    heapq.heappush(cand, (dj, j))
                    heapq.heappush(best, (-dj, j))
                    if len(best) > ef:
                        heapq.heappop(best)
        return sorted((-d, i) for d, i in best)

    def insert(self, v: Sequence[float]) -> int:
        x = np.asarray(v, dtype=np.float32)
        if x.shape != (self.dim,):
            raise ValueError(f"expected a vector of dimension {self.dim}")
        n = float(np.linalg.norm(x))
        x = x / n if n > 0 else x
        near = self._search(x, self.config.ef_construction)[: self.config.max_neighbors]
        idx = len(self.vectors)
        self.vectors.append(x)
        self.neighbors.append([i for _, i in near])
        for _, i in near:
            nb = self.neighbors[i]
            nb.append(idx)
            if len(nb) > self.config.max_neighbors:
                nb.sort(key=lambda j: self._dist(self.vectors[i], j))
                del nb[self.config.max_neighbors:]
        return idx

    def search(self, v: Sequence[float], k: int = 1) -> list[NswSearchResult]:
        x = np.asarray(v, dtype=np.float32)
        n = float(np.linalg.norm(x))
        x = x / n if n > 0 else x
        return [NswSearchResult(i, d) for d, i in self._search(x, max(self.config.ef_search, k))[:k]]


class EmbeddingIndex(Generic[T]):
    def __init__(self, dim: int, config: NswConfig | None = None):
        self.index = NswIndex(dim, config)
        self.payloads: list[T] = []

    def insert(self, v: Sequence[float], payload: T) -> int:
        i = self.index.insert(v)
        self.payloads.append(payload)
        return i

    def search(self, v: Sequence[float], k: int = 1) -> list[tuple[T, float]]:
        return [(self.payloads[r.index], r.distance) for r in self.index.search(v, k)]

    def __len__(self) -> int:
        return len(self.payloads)


@dataclass
class SemanticCacheConfig:
    similarity_threshold: float = 0.95
    capacity: int = 4096
    ttl: float | None = 600.0


class SemanticCache:
    """Answers a request whose embedding is close enough to a cached one."""

    def __init__(self, embed: Callable[[str], Sequence[float]], dim: int, config: SemanticCacheConfig | None = None):
        self.embed, self.config = embed, config or SemanticCacheConfig()
        self._idx: EmbeddingIndex[CachedResponse] = EmbeddingIndex(dim)
        self.hits = self.misses = 0

    def lookup(self, prompt: str) -> str | None:
        res = self._idx.search(self.embed(prompt), 1)
        if res and 1.0 - res[0][1] >= self.config.similarity_threshold and not res[0][0].is_expired():
            res[0][0].hits += 1
            self.hits += 1
            return res[0][0].text
        self.misses += 1
        return None

    def insert(self, prompt: str, response: str) -> None:
        if len(self._idx) < self.config.capacity:
            self._idx.insert(self.embed(prompt), CachedResponse(response, ttl=self.config.ttl))

    def __len__(self) -> int:
        return len(self._idx)

    def stats(self) -> dict:
        n = self.hits + self.misses
        return {"entries": len(self), "hits": self.hits, "misses": self.misses, "hit_rate": self.hits / n if n else 0.0}

    def run_or_cache(self, prompt: str, run: Callable[[str], str]) -> tuple[str, bool]:
        hit = self.lookup(prompt)
        if hit is not None:
            return hit, True
        out = run(prompt)
        self.insert(prompt, out)
        return out, False

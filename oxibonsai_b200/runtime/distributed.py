"""Request routing across engine replicas: consistent-hash ring, node registry with health and load, coordinator, and a
data-parallel replica pool for one multi-GPU box; plus the asyncio front of an engine.

Reference: crates/oxibonsai-runtime/src/distributed.rs:33-420 (FNV-1a ``ConsistentHashRing`` with virtual nodes,
``NodeRegistry`` health / load, ``DistributedCoordinator`` - in-memory only, "no actual TCP connections") and
async_engine.rs:26-154 (``AsyncInferenceEngine``: a semaphore bounding concurrent generations run on blocking threads).
``ReplicaPool`` is the per-GPU replica mode: one engine (or scheduler) per device, requests routed by session key so a
conversation keeps hitting the replica that holds its prefix cache, falling back to the least loaded healthy one.
"""
from __future__ import annotations

import asyncio
import bisect
import threading
from dataclasses import dataclass, field
from typing import Any, Callable, Iterator


def fnv1a_hash(data: bytes | str) -> int:
    if isinstance(data, str):
        data = data.encode("utf-8")
    h = 0xCBF29CE484222325
    for b in data:
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def _ring_hash(data: str) -> int:
    """FNV-1a followed by a 64-bit finaliser: plain FNV of near-identical short strings ("n0#1", "n0#2") clusters on the
    ring, the extra mixing spreads the virtual nodes evenly."""
    z = fnv1a_hash(data)
    z = ((z ^ (z >> 33)) * 0xFF51AFD7ED558CCD) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 33)) * 0xC4CEB9FE1A85EC53) & 0xFFFFFFFFFFFFFFFF
    return z ^ (z >> 33)


class ConsistentHashRing:
    def __init__(self, vnodes_per_node: int = 64):
        self.vnodes_per_node = vnodes_per_node
        self._keys: list[int] = []
        self._owner: dict[int, str] = {}
        self._nodes: set[str] = set()

    def add_node(self, node: str) -> None:
        if node in self._nodes:
            return
        self._nodes.add(node)
        for i in range(self.vnodes_per_node):
            k = _ring_hash(f"{node}#{i}")
            if k not in self._owner:
                bisect.insort(self._keys, k)
                self._owner[k] = node

    def remove_node(self, node: str) -> None:
        if node not in self._nodes:
            return
        self._nodes.discard(node)
        dead = [k for k, n in self._owner.items() if n == node]
        for k in dead:
            del self._owner[k]
        self._keys = sorted(self._owner)

    def get_node(self, key: str) -> str | None:
        if not self._keys:
            return None
        i = bisect.bisect_right(self._keys, _ring_hash(key)) % len(self._keys)
        return self._owner[self._keys[i]]

    def get_nodes(self, key: str, n: int) -> list[str]:
        """The first ``n`` distinct nodes clockwise from the key (for replication / fallback)."""
        out: list[str] = []
        if not self._keys:
            return out
        start = bisect.bisect_right(self._keys, _ring_hash(key))
        for j in range(len(self._keys)):
            node = self._owner[self._keys[(start + j) % len(self._keys)]]
            if node not in out:
                out.append(node)
                if len(out) == n:
                    break
        return out

    def node_count(self) -> int:
        return len(self._nodes)

    def vnode_count(self) -> int:
        return len(self._keys)


@dataclass
class NodeInfo:
    node_id: str
    address: str = ""
    healthy: bool = True
    load: float = 0.0
    capacity: int = 64
    meta: dict = field(default_factory=dict)


class NodeRegistry:
    def __init__(self, vnodes_per_node: int = 64):
        self.ring = ConsistentHashRing(vnodes_per_node)
        self._nodes: dict[str, NodeInfo] = {}
        self._lock = threading.Lock()

    def register(self, info: NodeInfo) -> None:
        with self._lock:
            self._nodes[info.node_id] = info
            self.ring.add_node(info.node_id)

    def deregister(self, node_id: str) -> bool:
        with self._lock:
            self.ring.remove_node(node_id)
            return self._nodes.pop(node_id, None) is not None

    def mark_healthy(self, node_id: str, healthy: bool) -> None:
        self._nodes[node_id].healthy = healthy

    def update_load(self, node_id: str, load: float) -> None:
        self._nodes[node_id].load = load

    def route_request(self, key: str, overload: float = 0.9) -> NodeInfo | None:
        """Hash owner when healthy and not overloaded, else the next ring nodes, else the least loaded healthy node."""
        for nid in self.ring.get_nodes(key, max(1, self.ring.node_count())):
            n = self._nodes.get(nid)
            if n is not None and n.healthy and n.load < overload:
                return n
        healthy = self.healthy_nodes()
        return min(healthy, key=lambda n: n.load) if healthy else None

    def healthy_nodes(self) -> list[NodeInfo]:
        return [n for n in self._nodes.values() if n.healthy]

    def all_nodes(self) -> list[NodeInfo]:
        return list(self._nodes.values())


@dataclass
class CoordinatorConfig:
    node_id: str = "local"
    address: str = "127.0.0.1:8080"
    vnodes_per_node: int = 64

    @classmethod
    def local_default(cls) -> "CoordinatorConfig":
        return cls()


class DistributedCoordinator:
    def __init__(self, config: CoordinatorConfig | None = None):
        self.config = config or CoordinatorConfig.local_default()
        self.registry = NodeRegistry(self.config.vnodes_per_node)

    def register_self(self) -> None:
        self.registry.register(NodeInfo(self.config.node_id, self.config.address))

    def add_peer(self, node_id: str, address: str, capacity: int = 64) -> None:
        self.registry.register(NodeInfo(node_id, address, capacity=capacity))

    def route(self, key: str) -> NodeInfo | None:
        return self.registry.route_request(key)

    def cluster_size(self) -> int:
        return len(self.registry.all_nodes())

    def healthy_count(self) -> int:
        return len(self.registry.healthy_nodes())

    def set_peer_health(self, node_id: str, healthy: bool) -> None:
        self.registry.mark_healthy(node_id, healthy)

    def update_peer_load(self, node_id: str, load: float) -> None:
        self.registry.update_load(node_id, load)

    def topology_summary(self) -> str:
        return "; ".join(f"{n.node_id}@{n.address} {'up' if n.healthy else 'down'} load={n.load:.2f}" for n in self.registry.all_nodes())


class ReplicaPool:
    """One backend per GPU behind the registry.  ``backends[node_id]`` must offer ``submit(...)`` like the scheduler."""

    def __init__(self, backends: dict[str, Any], capacity: int = 64):
        self.backends = backends
        self.registry = NodeRegistry()
        self._inflight = {k: 0 for k in backends}
        self._cap = capacity
        self._lock = threading.Lock()
        for k in backends:
            self.registry.register(NodeInfo(k, capacity=capacity))

    def pick(self, session_key: str) -> str:
        n = self.registry.route_request(session_key)
        if n is None:
            raise RuntimeError("no healthy replica")
        return n.node_id

    def submit(self, session_key: str, *args, **kw):
        nid = self.pick(session_key)
        with self._lock:
            self._inflight[nid] += 1
            self.registry.update_load(nid, self._inflight[nid] / self._cap)
        try:
            return nid, self.backends[nid].submit(*args, **kw)
        except Exception:
            self.registry.mark_healthy(nid, False)
            self.finished(nid)
            raise

    def finished(self, node_id: str) -> None:
        with self._lock:
            self._inflight[node_id] = max(0, self._inflight[node_id] - 1)
            self.registry.update_load(node_id, self._inflight[node_id] / self._cap)


class AsyncInferenceEngine:
    """asyncio front: at most ``max_concurrent`` generations in flight, each on a worker thread."""

    def __init__(self, generate: Callable[..., list[int]], stream: Callable[..., Iterator[int]] | None = None, max_concurrent: int = 8):
        self._generate, self._stream = generate, stream
        self._max = max_concurrent
        self._sem: asyncio.Semaphore | None = None
        self._active = 0

    def _semaphore(self) -> asyncio.Semaphore:
        if self._sem is None:
            self._sem = asyncio.Semaphore(self._max)
        return self._sem

    async def generate(self, *args, **kw) -> list[int]:
        async with self._semaphore():
            self._active += 1
            try:
                return await asyncio.get_running_loop().run_in_executor(None, lambda: self._generate(*args, **kw))
            finally:
                self._active -= 1

    async def generate_streaming(self, *args, **kw):
        if self._stream is None:
            raise RuntimeError("no streaming function configured")
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        done = object()

        def work():
            try:
                for tok in self._stream(*args, **kw):
                    loop.call_soon_threadsafe(q.put_nowait, tok)
                loop.call_soon_threadsafe(q.put_nowait, done)
            except Exception as e:  # delivered to the consumer
                loop.call_soon_threadsafe(q.put_nowait, e)
        async with self._semaphore():
            self._active += 1
            try:
                fut = loop.run_in_executor(None, work)
                while True:
                    item = await q.get()
                    if item is done:
                        break
                    if isinstance(item, Exception):
                        raise item
                    yield item
                await fut
            finally:
                self._active -= 1

    def active_requests(self) -> int:
        return self._active

    def max_concurrent(self) -> int:
        return self._max

    def has_capacity(self) -> bool:
        return self._active < self._max

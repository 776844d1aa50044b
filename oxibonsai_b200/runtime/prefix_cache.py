"""Prefix cache: a trie of token blocks mapping to KV pages, shared between sequences by reference counting.

Reference: ``PrefixCache`` (crates/oxibonsai-model/src/prefix_cache.rs:19-365: token-id trie of KV blocks, LRU by a
generation counter, hit-rate statistics), its session API ``PrefixAwarePrefill`` (:436-600) and the engine wrapper
(crates/oxibonsai-runtime/src/prefix_cache_engine.rs:59-250: look up, inject the cached blocks, prefill the suffix, store
the new blocks).  The reference copies cached f32 blocks into a fresh cache; with a paged KV pool nothing is copied -
a hit simply puts the cached page ids into the new sequence's block table and bumps their reference counts.  Only full
pages are shared (a sequence keeps appending into its own last page), and at least the last prompt token is always
recomputed because its logits are needed.
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass, field
from typing import Callable, Sequence


@dataclass
class _Node:
    page: int
    parent: "_Node | None"
    key: tuple
    children: dict = field(default_factory=dict)
    last_used: int = 0


@dataclass
class PrefixCacheStats:
    lookups: int = 0
    hits: int = 0
    tokens_requested: int = 0
    tokens_reused: int = 0
    inserted_pages: int = 0
    evicted_pages: int = 0

    @property
    def hit_rate(self) -> float:
        return self.hits / self.lookups if self.lookups else 0.0

    @property
    def token_reuse_rate(self) -> float:
        return self.tokens_reused / self.tokens_requested if self.tokens_requested else 0.0


class PrefixCache:
    """``retain(pages)`` / ``release(pages)`` adjust the page pool's reference counts."""

    def __init__(self, page_size: int, max_pages: int, retain: Callable[[list[int]], None], release: Callable[[list[int]], None]):
        self.page_size, self.max_pages = page_size, max_pages
        self._retain, self._release = retain, release
        self.root = _Node(-1, None, ())
        self.size = 0
        self.generation = 0
        self.stats = PrefixCacheStats()
        # Eviction candidates: (last_used, serial, node) for every node that was a leaf when it was last touched.  Entries are
        # not removed when a node gains a child, is used again or is evicted; one that no longer describes its node is
        # skipped when it comes up, so that an eviction costs O(log n) instead of a walk over the trie.
        self._heap: list[tuple[int, int, _Node]] = []
        self._serial = 0

    def _blocks(self, tokens: Sequence[int]):
        ps = self.page_size
        for i in range(len(tokens) // ps):
            yield tuple(tokens[i * ps:(i + 1) * ps])

    def lookup(self, tokens: Sequence[int], max_tokens: int | None = None) -> list[int]:
        """Pages of the longest cached prefix made of full blocks, covering at most ``max_tokens`` tokens."""
        self.generation += 1
        self.stats.lookups += 1
        self.stats.tokens_requested += len(tokens)
        limit = len(tokens) if max_tokens is None else max_tokens
        node, pages = self.root, []
        for blk in self._blocks(tokens):
            if (len(pages) + 1) * self.page_size > limit:
                break
            nxt = node.children.get(blk)
            if nxt is None:
                break
            nxt.last_used = self.generation
            pages.append(nxt.page)
            node = nxt
        if pages:
            self._candidate(node)
            self.stats.hits += 1
            self.stats.tokens_reused += len(pages) * self.page_size
        return pages

    def insert(self, tokens: Sequence[int], pages: Sequence[int]) -> int:
        """Records the full blocks of ``tokens`` as living in ``pages`` (page i holds block i).  Returns how many new
        pages the cache now references."""
        self.generation += 1
        node, added = self.root, 0
        for i, blk in enumerate(self._blocks(tokens)):
            if i >= len(pages):
                break
            nxt = node.children.get(blk)
            if nxt is None:
                if self.size >= self.max_pages and not self._evict_one(protect=node):
                    break
                nxt = _Node(int(pages[i]), node, blk)
                node.children[blk] = nxt
                self._retain([nxt.page])
                self.size += 1
                added += 1
            nxt.last_used = self.generation
            node = nxt
        self._candidate(node)
        self.stats.inserted_pages += added
        return added

    def _candidate(self, node: _Node) -> None:
        if node is self.root or node.children:
            return
        self._serial += 1
        heapq.heappush(self._heap, (node.last_used, self._serial, node))
        if len(self._heap) > 4 * self.size + 1024:                 # mostly entries of nodes that were used again: start over
            self._heap = [(n.last_used, i, n) for i, n in enumerate(self._leaves())]
            self._serial = len(self._heap)
            heapq.heapify(self._heap)

    def _leaves(self):
        stack = [self.root]
        while stack:
            n = stack.pop()
            if n is not self.root and not n.children:
                yield n
            stack.extend(n.children.values())

    def _evict_one(self, protect: _Node | None = None) -> bool:
        """Drops the least recently used leaf other than ``protect``."""
        victim, held = None, None
        while self._heap:
            entry = heapq.heappop(self._heap)
            used, _, n = entry
            if n.children or used != n.last_used or n.parent is None or n.parent.children.get(n.key) is not n:
                continue                                           # gained a child, was used again, or is gone
            if n is protect:
                held = entry
                continue
            victim = n
            break
        if held is not None:
            heapq.heappush(self._heap, held)
        if victim is None:
            return False
        parent = victim.parent
        del parent.children[victim.key]
        victim.parent = None
        self._release([victim.page])
        self.size -= 1
        self.stats.evicted_pages += 1
        self._candidate(parent)                                    # its last child went: it is a leaf now
        return True

    def evict(self, n_pages: int) -> int:
        """Drops up to ``n_pages`` least recently used leaf pages (called when the pool runs out of free pages)."""
        done = 0
        while done < n_pages and self._evict_one():
            done += 1
        return done

    def clear(self) -> None:
        while self._evict_one():
            pass

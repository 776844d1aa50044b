"""The Earley recogniser and the vocabulary mask in C++ (csrc/runtime/grammar_matcher.cpp).

Reference: crates/oxibonsai-runtime/src/grammar/earley.rs:39-193, constraint.rs:66, cache.rs:52.  ``NativeEarley`` has the
interface of the Python :class:`~oxibonsai_b200.runtime.grammar.earley.EarleyRecognizer` (which stays as the oracle of the
tests) plus ``mask``: the packed allowed-token mask at the current position, found by walking the vocabulary's byte trie
with one recogniser and cached per chart signature inside the compiled grammar, so every matcher of a grammar - every
request with the same ``response_format`` - shares the finished masks.
"""
from __future__ import annotations

import ctypes as C
import threading
from collections import OrderedDict

import numpy as np

from ... import _native
from .ast import Grammar, Term


def _lib():
    lib = _native.host()
    if "bgram_compile" not in lib._declared:
        vp, u32, i32 = C.c_void_p, C.c_uint32, C.c_int32
        _native.declare(lib, {"bgram_compile": (vp, [vp, u32]), "bgram_free": (None, [vp]), "bgram_matcher_new": (vp, [vp]),
                              "bgram_matcher_free": (None, [vp]), "bgram_matcher_reset": (None, [vp]), "bgram_matcher_feed": (C.c_int, [vp, C.c_char_p, u32]),
                              "bgram_matcher_complete": (C.c_int, [vp]), "bgram_matcher_dead": (C.c_int, [vp]), "bgram_matcher_position": (u32, [vp]),
                              "bgram_matcher_signature": (C.c_uint64, [vp]), "bgram_matcher_items": (u32, [vp]), "bgram_matcher_next_bytes": (None, [vp, vp]),
                              "bgram_matcher_mask": (u32, [vp, vp, i32, vp, vp]), "bgram_cache_stats": (None, [vp, vp])})
        lib._declared.add("bgram_compile")
    return lib


def serialize(grammar: Grammar) -> np.ndarray:
    """The grammar as the int32 blob ``bgram_compile`` reads: terminal byte sets first, then the alternatives of every rule."""
    grammar.validate()
    names = list(grammar.rules)
    idx = {n: i for i, n in enumerate(names)}
    terms: dict[frozenset, int] = {}

    def code(s) -> int:
        return -(terms.setdefault(s.bytes, len(terms)) + 1) if isinstance(s, Term) else idx[s.name]
    # a production holds at most 255 symbols natively: longer ones continue in helper rules appended after the named ones
    rules: list[list[list[int]]] = [[] for _ in names]
    for r, n in enumerate(names):
        for alt in grammar.rules[n].alternatives:
            syms = [code(s) for s in alt]
            target = r
            while len(syms) > 200:
                helper = len(rules)
                rules.append([])
                rules[target].append(syms[:200] + [helper])
                syms, target = syms[200:], helper
            rules[target].append(syms)
    body: list[int] = []
    for alts in rules:
        body.append(len(alts))
        for syms in alts:
            body.append(len(syms))
            body += syms
    words: list[int] = []
    for bs in terms:                                   # insertion order = id order
        bits = 0
        for b in bs:
            bits |= 1 << b
        words += [(bits >> (32 * k)) & 0xFFFFFFFF for k in range(8)]
    head = [len(terms), len(rules), idx[grammar.start]]
    return np.asarray(head + words + body, dtype=np.int64).astype(np.uint32).view(np.int32)


class CompiledGrammar:
    """A grammar compiled once; holds the mask cache that its matchers share."""

    def __init__(self, grammar: Grammar):
        self._lib = _lib()
        blob = serialize(grammar)
        self.key = blob.tobytes()
        self._h = self._lib.bgram_compile(blob.ctypes.data, blob.size)
        if not self._h:
            raise ValueError("the grammar could not be compiled (a production longer than 255 symbols, or a malformed rule)")

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.bgram_free(self._h)
            self._h = None

    def cache_stats(self) -> dict:
        out = (C.c_uint64 * 6)()
        self._lib.bgram_cache_stats(self._h, out)
        return {"hits": int(out[0]), "misses": int(out[1]), "entries": int(out[2]), "transitions": int(out[3]),
                "edges_through_recogniser": int(out[4]), "edges_through_automaton": int(out[5])}


_COMPILED: "OrderedDict[bytes, CompiledGrammar]" = OrderedDict()
_COMPILED_LOCK = threading.Lock()
_COMPILED_CAP = 32


def compile_cached(grammar: Grammar) -> CompiledGrammar:
    """Structurally equal grammars share one compiled object, and with it the masks computed so far (an LRU of 32; a grammar keeps at most 32 MB of masks)."""
    key = serialize(grammar).tobytes()
    with _COMPILED_LOCK:
        cg = _COMPILED.get(key)
        if cg is not None:
            _COMPILED.move_to_end(key)
            return cg
    cg = CompiledGrammar(grammar)
    with _COMPILED_LOCK:
        _COMPILED[key] = cg
        while len(_COMPILED) > _COMPILED_CAP:
            _COMPILED.popitem(last=False)
    return cg


class NativeEarley:
    def __init__(self, grammar: Grammar | CompiledGrammar):
        self.compiled = grammar if isinstance(grammar, CompiledGrammar) else compile_cached(grammar)
        self._lib = self.compiled._lib
        self._h = self._lib.bgram_matcher_new(self.compiled._h)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.bgram_matcher_free(self._h)
            self._h = None

    @property
    def dead(self) -> bool:
        return bool(self._lib.bgram_matcher_dead(self._h))

    @property
    def position(self) -> int:
        return int(self._lib.bgram_matcher_position(self._h))

    def reset(self) -> None:
        self._lib.bgram_matcher_reset(self._h)

    def feed(self, byte: int) -> bool:
        return bool(self._lib.bgram_matcher_feed(self._h, bytes([byte & 0xFF]), 1))

    def feed_bytes(self, data: bytes) -> bool:
        return bool(self._lib.bgram_matcher_feed(self._h, bytes(data), len(data)))

    def is_complete(self) -> bool:
        return bool(self._lib.bgram_matcher_complete(self._h))

    def next_bytes(self) -> frozenset[int]:
        out = np.zeros(256, dtype=np.uint8)
        self._lib.bgram_matcher_next_bytes(self._h, out.ctypes.data)
        return frozenset(int(b) for b in np.flatnonzero(out))

    def signature(self) -> int:
        return int(self._lib.bgram_matcher_signature(self._h))

    def item_count(self) -> int:
        return int(self._lib.bgram_matcher_items(self._h))

    def accepts(self, data: bytes) -> bool:
        m = NativeEarley(self.compiled)
        return m.feed_bytes(data) and m.is_complete()

    def mask(self, table, eos_token: int | None = None) -> tuple[np.ndarray, bool]:
        """(packed mask of the tokens that may come next, whether it came from the cache)."""
        mask = np.zeros(table.words, dtype=np.uint32)
        cached = C.c_int(0)
        self._lib.bgram_matcher_mask(self._h, table._h, -1 if eos_token is None else int(eos_token), mask.ctypes.data, C.byref(cached))
        return mask, bool(cached.value)

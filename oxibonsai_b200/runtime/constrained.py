"""Constrained decoding: token constraints, vocabulary masks and the sampler wrapper that applies them.

Reference: crates/oxibonsai-runtime/src/constrained_decoding/error_trait.rs:14-63 (``TokenConstraint``:
``allowed_tokens`` / ``advance`` / ``is_complete`` / ``reset`` / ``name``), sampler.rs:19-94 (``ConstrainedSampler`` masks the
logits before sampling), allow_list.rs, sequence.rs, length.rs, regex.rs, json.rs, and grammar/constraint.rs:66 +
grammar/cache.rs:52 (``GrammarConstraint`` with an ``AllowedTokensCache``).

Masks are packed 32 tokens per uint32 (bit set = allowed): exactly what the GPU sampler's ``allow_mask`` argument takes,
so a constraint costs one small host-to-device copy per token and no extra kernel.  The per-token automaton walk over
the vocabulary runs in C++ (csrc/runtime/token_mask.cpp for automata, csrc/runtime/grammar_matcher.cpp for grammars).
"""
from __future__ import annotations

import ctypes as C
from collections import OrderedDict
from typing import Callable, Iterable, Sequence

import numpy as np

from .. import _native
from .grammar.ast import Grammar
from .grammar.earley import EarleyRecognizer
from .grammar.regex_compiler import Dfa, compile_regex


def _lib():
    lib = _native.host()
    if "btok_new" not in lib._declared:
        vp, u32 = C.c_void_p, C.c_uint32
        _native.declare(lib, {"btok_new": (vp, [vp, vp, u32]), "btok_free": (None, [vp]), "btok_count": (u32, [vp]),
                              "btok_dfa_mask": (u32, [vp, vp, C.c_int32, C.c_int32, vp, vp]),
                              "btok_candidates": (u32, [vp, vp, vp, u32]), "btok_pack_ids": (None, [vp, u32, u32, vp])})
        lib._declared.add("btok_new")
    return lib


class TokenTable:
    """Byte strings of the whole vocabulary, held natively."""

    def __init__(self, token_bytes: Sequence[bytes]):
        self.tokens = [bytes(t) for t in token_bytes]
        self.n = len(self.tokens)
        off = np.zeros(self.n + 1, dtype=np.uint32)
        off[1:] = np.cumsum([len(t) for t in self.tokens])
        blob = np.frombuffer(b"".join(self.tokens) or b"\0", dtype=np.uint8)
        self._lib = _lib()
        self._h = self._lib.btok_new(off.ctypes.data, blob.ctypes.data, self.n)
        self.words = (self.n + 31) // 32

    @classmethod
    def from_tokenizer(cls, tokenizer, vocab_size: int | None = None) -> "TokenTable":
        n = vocab_size or tokenizer.vocab_size
        return cls([tokenizer.token_bytes(i) for i in range(n)])

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.btok_free(self._h)
            self._h = None

    def dfa_mask(self, dfa: Dfa, state: int) -> tuple[np.ndarray, np.ndarray]:
        mask = np.zeros(self.words, dtype=np.uint32)
        nxt = np.full(self.n, -1, dtype=np.int32)
        trans = np.ascontiguousarray(dfa.trans, dtype=np.int32)
        self._lib.btok_dfa_mask(self._h, trans.ctypes.data, dfa.n_states, int(state), mask.ctypes.data, nxt.ctypes.data)
        return mask, nxt

    def candidates(self, first_bytes: Iterable[int]) -> np.ndarray:
        ok = np.zeros(256, dtype=np.uint8)
        ok[list(first_bytes)] = 1
        out = np.empty(self.n, dtype=np.uint32)
        k = self._lib.btok_candidates(self._h, ok.ctypes.data, out.ctypes.data, self.n)
        return out[:k]

    def pack(self, ids: Iterable[int]) -> np.ndarray:
        arr = np.fromiter((int(i) for i in ids), dtype=np.uint32)
        mask = np.zeros(self.words, dtype=np.uint32)
        self._lib.btok_pack_ids(arr.ctypes.data if arr.size else None, arr.size, self.n, mask.ctypes.data)
        return mask


def mask_to_bool(mask: np.ndarray, n: int) -> np.ndarray:
    return np.unpackbits(mask.view(np.uint8), bitorder="little")[:n].astype(bool)


# ---- constraints -------------------------------------------------------------------------------------------------------------
class TokenConstraint:
    """Base protocol.  ``allowed_mask`` returns a packed mask or None for "everything allowed"."""
    name = "constraint"

    def allowed_mask(self) -> np.ndarray | None:
        return None

    def allowed_tokens(self, vocab_size: int) -> np.ndarray | None:
        m = self.allowed_mask()
        return None if m is None else mask_to_bool(m, vocab_size)

    def advance(self, token: int) -> bool:
        return True

    def is_complete(self) -> bool:
        """Whether the output so far is a valid place to stop (a terminal state)."""
        return True

    def finished(self) -> bool:
        """Whether the generation has to end here: the constraint's language admits no useful continuation.  Engines and
        the scheduler end a constrained sequence on this, on EOS and on the token limit; an always-terminal constraint
        (an allow-list, a length window) never asks for the end itself."""
        return False

    def reset(self) -> None:
        pass


class NoConstraint(TokenConstraint):
    name = "none"


class AllowListConstraint(TokenConstraint):
    name = "allow_list"

    def __init__(self, table: TokenTable, allowed: Iterable[int]):
        self.ids = sorted(set(int(i) for i in allowed))
        self._mask = table.pack(self.ids)

    def allowed_mask(self):
        return self._mask

    def advance(self, token: int) -> bool:
        return token in set(self.ids)


class SequenceConstraint(TokenConstraint):
    """Forces an exact token sequence; the generation ends after its last token (a caller that keeps sampling past it gets
    every token allowed)."""
    name = "sequence"

    def __init__(self, table: TokenTable, sequence: Sequence[int]):
        self.table, self.seq, self.pos = table, [int(t) for t in sequence], 0

    def allowed_mask(self):
        return self.table.pack([self.seq[self.pos]]) if self.pos < len(self.seq) else None

    def advance(self, token: int) -> bool:
        if self.pos < len(self.seq):
            if token != self.seq[self.pos]:
                return False
            self.pos += 1
        return True

    def is_complete(self) -> bool:
        return self.pos >= len(self.seq)

    def finished(self) -> bool:
        return self.pos >= len(self.seq)

    def reset(self) -> None:
        self.pos = 0


class LengthConstraint(TokenConstraint):
    """EOS is forbidden before ``min_tokens`` and forced at ``max_tokens``."""
    name = "length"

    def __init__(self, table: TokenTable, eos_token: int, min_tokens: int = 0, max_tokens: int | None = None):
        self.table, self.eos, self.lo, self.hi, self.count = table, eos_token, min_tokens, max_tokens, 0
        full = np.full(table.words, 0xFFFFFFFF, dtype=np.uint32)
        if table.n % 32:
            full[-1] = (1 << (table.n % 32)) - 1
        self._no_eos = full.copy()
        if 0 <= eos_token < table.n:
            self._no_eos[eos_token >> 5] &= ~np.uint32(1 << (eos_token & 31))

    def allowed_mask(self):
        if self.hi is not None and self.count >= self.hi:
            return self.table.pack([self.eos])
        return self._no_eos if self.count < self.lo else None

    def advance(self, token: int) -> bool:
        self.count += 1
        return True

    def is_complete(self) -> bool:
        return self.count >= self.lo

    def reset(self) -> None:
        self.count = 0


class DfaConstraint(TokenConstraint):
    """Output must match a byte-level DFA (a compiled regular expression); EOS is allowed in accepting states."""
    name = "regex"

    def __init__(self, table: TokenTable, dfa: Dfa, eos_token: int | None = None, cache_size: int = 4096):
        self.table, self.dfa, self.eos, self.state = table, dfa, eos_token, 0
        self._cache: OrderedDict[int, tuple[np.ndarray, np.ndarray]] = OrderedDict()
        self._cap = cache_size
        self.cache_hits = self.cache_misses = 0

    @classmethod
    def from_regex(cls, table: TokenTable, pattern: str, eos_token: int | None = None) -> "DfaConstraint":
        return cls(table, compile_regex(pattern), eos_token)

    def _entry(self, state: int):
        e = self._cache.get(state)
        if e is not None:
            self._cache.move_to_end(state)
            self.cache_hits += 1
            return e
        self.cache_misses += 1
        mask, nxt = self.table.dfa_mask(self.dfa, state)
        if self.eos is not None and self.dfa.accepting[state] and 0 <= self.eos < self.table.n:
            mask[self.eos >> 5] |= np.uint32(1 << (self.eos & 31))
        self._cache[state] = (mask, nxt)
        if len(self._cache) > self._cap:
            self._cache.popitem(last=False)
        return mask, nxt

    def allowed_mask(self):
        if self.state < 0:
            return np.zeros(self.table.words, dtype=np.uint32)
        return self._entry(self.state)[0]

    def advance(self, token: int) -> bool:
        if self.eos is not None and token == self.eos:
            return self.is_complete()
        if self.state < 0:
            return False
        self.state = self.dfa.run(self.state, self.table.tokens[token]) if self.table.tokens[token] else -1
        return self.state >= 0

    def is_complete(self) -> bool:
        return self.state >= 0 and bool(self.dfa.accepting[self.state])

    def finished(self) -> bool:
        """Dead state, or an accepting state that no token other than EOS can leave."""
        if self.state < 0:
            return True
        if not self.dfa.accepting[self.state]:
            return False
        mask = self._entry(self.state)[0].copy()
        if self.eos is not None and 0 <= self.eos < self.table.n:
            mask[self.eos >> 5] &= ~np.uint32(1 << (self.eos & 31))
        return not mask.any()

    def reset(self) -> None:
        self.state = 0


class GrammarConstraint(TokenConstraint):
    """Output must be a sentence of a context-free grammar (Earley).  The recogniser and the search for the allowed tokens
    run in C++ (``grammar/native.py``): one recogniser walks the vocabulary's byte trie depth-first, entering only the bytes
    the grammar can scan, and the finished mask is cached under the chart position's signature inside the compiled grammar,
    which every constraint over a structurally equal grammar shares.  ``native=False`` selects the Python recogniser (the
    oracle of the tests)."""
    name = "grammar"

    def __init__(self, table: TokenTable, grammar: Grammar, eos_token: int | None = None, cache_size: int = 512, native: bool = True):
        self.table, self.eos, self.native = table, eos_token, native
        if native:
            from .grammar.native import NativeEarley
            self.rec = NativeEarley(grammar)
        else:
            self.rec = EarleyRecognizer(grammar)
        self.text = bytearray()
        self._cache: OrderedDict[bytes, np.ndarray] = OrderedDict()
        self._cap = cache_size
        self.cache_hits = 0

    def allowed_mask(self):
        if self.native:
            mask, cached = self.rec.mask(self.table, self.eos)
            self.cache_hits += int(cached)
            return mask
        key = bytes(self.text)
        if key in self._cache:
            self._cache.move_to_end(key)
            self.cache_hits += 1
            return self._cache[key]
        ok: list[int] = []
        cand = self.table.candidates(self.rec.next_bytes())
        memo: dict[bytes, EarleyRecognizer | None] = {b"": self.rec}

        def state_after(prefix: bytes):
            st = memo.get(prefix, 0)
            if st != 0:
                return st
            parent = state_after(prefix[:-1])
            if parent is None:
                memo[prefix] = None
                return None
            f = parent.fork()
            memo[prefix] = f if f.feed(prefix[-1]) else None
            return memo[prefix]
        for i in cand:
            if state_after(self.table.tokens[i]) is not None:
                ok.append(int(i))
        if self.eos is not None and self.rec.is_complete():
            ok.append(self.eos)
        mask = self.table.pack(ok)
        self._cache[key] = mask
        if len(self._cache) > self._cap:
            self._cache.popitem(last=False)
        return mask

    def advance(self, token: int) -> bool:
        if self.eos is not None and token == self.eos:
            return self.rec.is_complete()
        data = self.table.tokens[token]
        if not data or not self.rec.feed_bytes(data):
            return False
        self.text += data
        return True

    def is_complete(self) -> bool:
        return self.rec.is_complete()

    def finished(self) -> bool:
        """The first complete sentence ends the generation (a JSON value is returned as soon as it closes)."""
        return self.rec.is_complete()

    def reset(self) -> None:
        self.rec.reset()
        self.text = bytearray()


def json_constraint(table: TokenTable, eos_token: int | None = None) -> GrammarConstraint:
    from .grammar.compilers import json_grammar
    return GrammarConstraint(table, json_grammar(), eos_token)


def json_schema_constraint(table: TokenTable, schema, eos_token: int | None = None) -> GrammarConstraint:
    from .grammar.compilers import json_schema_to_grammar
    return GrammarConstraint(table, json_schema_to_grammar(schema), eos_token)


class AllOf(TokenConstraint):
    """Intersection of several constraints."""
    name = "all_of"

    def __init__(self, *constraints: TokenConstraint):
        self.cs = list(constraints)

    def allowed_mask(self):
        out = None
        for c in self.cs:
            m = c.allowed_mask()
            if m is not None:
                out = m.copy() if out is None else (out & m)
        return out

    def advance(self, token: int) -> bool:
        return all([c.advance(token) for c in self.cs])

    def is_complete(self) -> bool:
        return all(c.is_complete() for c in self.cs)

    def finished(self) -> bool:
        return any(c.finished() for c in self.cs) and self.is_complete()

    def reset(self) -> None:
        for c in self.cs:
            c.reset()


class ConstraintViolation(RuntimeError):
    pass


class ConstrainedSampler:
    """Wraps a ``sample(logits) -> token`` function: masks forbidden tokens to -inf, samples, advances the constraint."""

    def __init__(self, constraint: TokenConstraint, sample_fn: Callable[[np.ndarray], int], vocab_size: int):
        self.constraint, self.sample_fn, self.vocab = constraint, sample_fn, vocab_size
        self.masked_steps = 0

    def sample(self, logits: np.ndarray) -> int:
        allowed = self.constraint.allowed_tokens(self.vocab)
        x = np.asarray(logits, dtype=np.float64)
        if allowed is not None:
            if not allowed.any():
                raise ConstraintViolation(f"{self.constraint.name}: no token can continue the output")
            x = np.where(allowed[: len(x)], x, -np.inf)
            self.masked_steps += 1
        tok = int(self.sample_fn(x))
        if not self.constraint.advance(tok):
            raise ConstraintViolation(f"{self.constraint.name}: sampled token {tok} violates the constraint")
        return tok

    def gpu_mask(self) -> np.ndarray | None:
        """Packed mask for the device sampler (None = unconstrained step)."""
        return self.constraint.allowed_mask()

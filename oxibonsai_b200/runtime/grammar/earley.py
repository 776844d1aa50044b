"""Incremental byte-level Earley recogniser.

Reference: crates/oxibonsai-runtime/src/grammar/earley.rs:39-193 (``EarleyRecognizer`` with ``FirstSets``): feed one
byte at a time, ask which bytes may come next, ask whether the input so far is a complete sentence.  Nullable rules
are handled in the predictor (Aycock-Horspool), so empty productions need no special casing by callers.  ``fork()``
gives an independent recogniser sharing the immutable chart prefix, which is what the token-mask search uses to try
multi-byte tokens without disturbing the main state.
"""
from __future__ import annotations

from .ast import Grammar, Term


class EarleyRecognizer:
    def __init__(self, grammar: Grammar):
        grammar.validate()
        self.g = grammar
        self._names = list(grammar.rules)
        self._idx = {n: i for i, n in enumerate(self._names)}
        # productions as tuples: symbol = frozenset (terminal) or int (rule index)
        self._prods: list[list[tuple]] = []
        for n in self._names:
            alts = []
            for alt in grammar.rules[n].alternatives:
                alts.append(tuple(s.bytes if isinstance(s, Term) else self._idx[s.name] for s in alt))
            self._prods.append(alts)
        self._nullable = {self._idx[n] for n in grammar.nullable()}
        self._start = self._idx[grammar.start]
        self.chart: list[frozenset] = []
        self.dead = False
        self._begin()

    # an item is (rule, alt, dot, origin)
    def _close(self, items: set, pos: int) -> frozenset:
        work = list(items)
        seen = set(items)

        def push(it):
            if it not in seen:
                seen.add(it)
                work.append(it)
        while work:
            r, a, d, o = work.pop()
            prod = self._prods[r][a]
            if d < len(prod):
                sym = prod[d]
                if isinstance(sym, int):
                    for ai in range(len(self._prods[sym])):
                        push((sym, ai, 0, pos))
                    if sym in self._nullable:
                        push((r, a, d + 1, o))
            else:
                # completion: advance every item of the origin set waiting for rule r
                src = seen if o == pos else self.chart[o]
                for (r2, a2, d2, o2) in list(src):
                    p2 = self._prods[r2][a2]
                    if d2 < len(p2) and p2[d2] == r and isinstance(p2[d2], int):
                        push((r2, a2, d2 + 1, o2))
        return frozenset(seen)

    def _begin(self) -> None:
        self.chart = [self._close({(self._start, ai, 0, 0) for ai in range(len(self._prods[self._start]))}, 0)]
        self.dead = False

    def reset(self) -> None:
        self._begin()

    def fork(self) -> "EarleyRecognizer":
        c = object.__new__(EarleyRecognizer)
        c.__dict__.update(self.__dict__)
        c.chart = list(self.chart)
        return c

    @property
    def position(self) -> int:
        return len(self.chart) - 1

    def next_bytes(self) -> frozenset[int]:
        if self.dead:
            return frozenset()
        out: set[int] = set()
        for r, a, d, _ in self.chart[-1]:
            prod = self._prods[r][a]
            if d < len(prod) and not isinstance(prod[d], int):
                out |= prod[d]
        return frozenset(out)

    def feed(self, byte: int) -> bool:
        """Consumes one byte; returns False (and becomes dead) when no parse can continue."""
        if self.dead:
            return False
        pos = len(self.chart)
        scanned = set()
        for r, a, d, o in self.chart[-1]:
            prod = self._prods[r][a]
            if d < len(prod) and not isinstance(prod[d], int) and byte in prod[d]:
                scanned.add((r, a, d + 1, o))
        if not scanned:
            self.dead = True
            return False
        self.chart.append(frozenset())
        self.chart[pos] = self._close(scanned, pos)
        return True

    def feed_bytes(self, data: bytes) -> bool:
        return all(self.feed(b) for b in data)

    def is_complete(self) -> bool:
        if self.dead:
            return False
        return any(r == self._start and o == 0 and d == len(self._prods[r][a]) for r, a, d, o in self.chart[-1])

    def accepts(self, data: bytes) -> bool:
        f = self.fork()
        f.reset()
        return f.feed_bytes(data) and f.is_complete()

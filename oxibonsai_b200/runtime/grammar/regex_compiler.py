"""Regular expressions -> byte-level automata (Thompson NFA, subset construction to a DFA of bounded size).

Reference: crates/oxibonsai-runtime/src/grammar/regex_compiler.rs (regex -> Thompson NFA -> DFA with at most 2048
states, then a right-linear grammar) and constrained_decoding/regex.rs (the NFA-driven regex constraint).

Supported syntax: literals, ``.``, classes ``[a-z0-9_]`` / ``[^...]``, escapes ``\\d \\w \\s \\D \\W \\S \\n \\t \\r \\xHH`` and
escaped metacharacters, groups ``( )`` and ``(?: )``, alternation ``|``, quantifiers ``* + ? {m} {m,} {m,n}``.  Matching is
anchored at both ends and runs over UTF-8 bytes; a non-ASCII literal is the sequence of its bytes and ``.`` matches any
byte but a newline.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

MAX_DFA_STATES = 2048
_ALL = frozenset(range(256))
_DIGIT = frozenset(range(48, 58))
_WORD = frozenset(list(range(48, 58)) + list(range(65, 91)) + list(range(97, 123)) + [95])
_SPACE = frozenset(b" \t\n\r\f\v")


class RegexError(ValueError):
    pass


# ---- parser: pattern -> AST ----------------------------------------------------------------------------------------------
# AST nodes: ("set", frozenset[int]) | ("cat", [nodes]) | ("alt", [nodes]) | ("rep", node, lo, hi|None) | ("empty",)
class _Parser:
    def __init__(self, pattern: str):
        self.s, self.i = pattern, 0

    def parse(self):
        node = self._alt()
        if self.i != len(self.s):
            raise RegexError(f"unexpected {self.s[self.i]!r} at {self.i}")
        return node

    def _peek(self):
        return self.s[self.i] if self.i < len(self.s) else None

    def _alt(self):
        parts = [self._cat()]
        while self._peek() == "|":
            self.i += 1
            parts.append(self._cat())
        return parts[0] if len(parts) == 1 else ("alt", parts)

    def _cat(self):
        items = []
        while self._peek() is not None and self._peek() not in "|)":
            items.append(self._repeat())
        if not items:
            return ("empty",)
        return items[0] if len(items) == 1 else ("cat", items)

    def _repeat(self):
        atom = self._atom()
        while True:
            c = self._peek()
            if c == "*":
                self.i += 1
                atom = ("rep", atom, 0, None)
            elif c == "+":
                self.i += 1
                atom = ("rep", atom, 1, None)
            elif c == "?":
                self.i += 1
                atom = ("rep", atom, 0, 1)
            elif c == "{":
                j = self.s.find("}", self.i)
                body = self.s[self.i + 1:j] if j > 0 else ""
                parts = body.split(",")
                if j < 0 or not parts[0].isdigit() or len(parts) > 2 or (len(parts) == 2 and parts[1] and not parts[1].isdigit()):
                    raise RegexError(f"bad quantifier at {self.i}")
                lo = int(parts[0])
                hi = lo if len(parts) == 1 else (int(parts[1]) if parts[1] else None)
                if hi is not None and hi < lo or lo > 256 or (hi or 0) > 256:
                    raise RegexError("quantifier bounds out of range")
                self.i = j + 1
                atom = ("rep", atom, lo, hi)
            else:
                return atom
            if self._peek() == "?":      # lazy modifiers do not change the language
                self.i += 1

    def _escape(self) -> frozenset[int]:
        c = self._peek()
        if c is None:
            raise RegexError("dangling backslash")
        self.i += 1
        table = {"d": _DIGIT, "D": _ALL - _DIGIT, "w": _WORD, "W": _ALL - _WORD, "s": _SPACE, "S": _ALL - _SPACE,
                 "n": frozenset([10]), "t": frozenset([9]), "r": frozenset([13]), "f": frozenset([12]), "v": frozenset([11]), "0": frozenset([0])}
        if c in table:
            return table[c]
        if c == "x":
            h = self.s[self.i:self.i + 2]
            if len(h) != 2:
                raise RegexError("bad \\x escape")
            self.i += 2
            return frozenset([int(h, 16)])
        if ord(c) < 128:
            return frozenset([ord(c)])
        raise RegexError("escaped non-ASCII character")

    def _atom(self):
        c = self._peek()
        self.i += 1
        if c == "(":
            if self.s.startswith("?:", self.i):
                self.i += 2
            node = self._alt()
            if self._peek() != ")":
                raise RegexError("missing )")
            self.i += 1
            return node
        if c == "[":
            return ("set", self._cls())
        if c == ".":
            return ("set", _ALL - {10})
        if c == "\\":
            return ("set", self._escape())
        if c in "*+?{":
            raise RegexError(f"nothing to repeat at {self.i - 1}")
        if c in "^$":
            return ("empty",)            # matching is anchored anyway
        b = c.encode("utf-8")
        if len(b) == 1:
            return ("set", frozenset(b))
        return ("cat", [("set", frozenset([x])) for x in b])

    def _cls(self) -> frozenset[int]:
        neg = self._peek() == "^"
        if neg:
            self.i += 1
        out: set[int] = set()
        first = True
        while True:
            c = self._peek()
            if c is None:
                raise RegexError("missing ]")
            if c == "]" and not first:
                self.i += 1
                break
            first = False
            self.i += 1
            if c == "\\":
                s = self._escape()
                if len(s) != 1:
                    out |= s
                    continue
                lo = next(iter(s))
            else:
                if ord(c) > 127:
                    raise RegexError("non-ASCII character in a class")
                lo = ord(c)
            if self._peek() == "-" and self.i + 1 < len(self.s) and self.s[self.i + 1] != "]":
                self.i += 1
                h = self._peek()
                self.i += 1
                if h == "\\":
                    hs = self._escape()
                    if len(hs) != 1:
                        raise RegexError("bad range")
                    hi = next(iter(hs))
                else:
                    hi = ord(h)
                if hi < lo:
                    raise RegexError("reversed range")
                out |= set(range(lo, hi + 1))
            else:
                out.add(lo)
        return frozenset(_ALL - out) if neg else frozenset(out)


# ---- Thompson NFA ------------------------------------------------------------------------------------------------------------
@dataclass
class Nfa:
    eps: list[list[int]] = field(default_factory=list)
    trans: list[list[tuple[frozenset[int], int]]] = field(default_factory=list)
    start: int = 0
    accept: int = 0

    def new(self) -> int:
        self.eps.append([])
        self.trans.append([])
        return len(self.eps) - 1

    def closure(self, states) -> frozenset[int]:
        stack, seen = list(states), set(states)
        while stack:
            for t in self.eps[stack.pop()]:
                if t not in seen:
                    seen.add(t)
                    stack.append(t)
        return frozenset(seen)


def _build(nfa: Nfa, node) -> tuple[int, int]:
    kind = node[0]
    if kind == "empty":
        s = nfa.new()
        return s, s
    if kind == "set":
        s, e = nfa.new(), nfa.new()
        nfa.trans[s].append((node[1], e))
        return s, e
    if kind == "cat":
        s, e = _build(nfa, node[1][0])
        for n in node[1][1:]:
            s2, e2 = _build(nfa, n)
            nfa.eps[e].append(s2)
            e = e2
        return s, e
    if kind == "alt":
        s, e = nfa.new(), nfa.new()
        for n in node[1]:
            s2, e2 = _build(nfa, n)
            nfa.eps[s].append(s2)
            nfa.eps[e2].append(e)
        return s, e
    if kind == "rep":
        _, inner, lo, hi = node
        s = e = nfa.new()
        for _ in range(lo):
            s2, e2 = _build(nfa, inner)
            nfa.eps[e].append(s2)
            e = e2
        if hi is None:
            s2, e2 = _build(nfa, inner)
            nfa.eps[e].append(s2)
            nfa.eps[e2].append(s2)
            out = nfa.new()
            nfa.eps[e].append(out)
            nfa.eps[e2].append(out)
            e = out
        else:
            out = nfa.new()
            for _ in range(hi - lo):
                s2, e2 = _build(nfa, inner)
                nfa.eps[e].append(s2)
                nfa.eps[e].append(out)
                e = e2
            nfa.eps[e].append(out)
            e = out
        return s, e
    raise RegexError(f"unknown node {kind}")


def regex_to_nfa(pattern: str) -> Nfa:
    nfa = Nfa()
    nfa.start, nfa.accept = _build(nfa, _Parser(pattern).parse())
    return nfa


# ---- DFA -------------------------------------------------------------------------------------------------------------------------
@dataclass
class Dfa:
    """``trans[state, byte]`` is the next state or -1; state 0 is the start."""
    trans: np.ndarray               # int32 [n_states, 256]
    accepting: np.ndarray           # bool [n_states]

    @property
    def n_states(self) -> int:
        return self.trans.shape[0]

    def step(self, state: int, byte: int) -> int:
        return int(self.trans[state, byte]) if state >= 0 else -1

    def run(self, state: int, data: bytes) -> int:
        for b in data:
            if state < 0:
                return -1
            state = int(self.trans[state, b])
        return state

    def matches(self, data: bytes) -> bool:
        s = self.run(0, data)
        return s >= 0 and bool(self.accepting[s])

    def next_bytes(self, state: int) -> np.ndarray:
        return np.flatnonzero(self.trans[state] >= 0) if state >= 0 else np.empty(0, dtype=np.int64)

    def live_states(self) -> np.ndarray:
        """States from which an accepting state is reachable."""
        n = self.n_states
        live = self.accepting.copy()
        changed = True
        while changed:
            nxt = self.trans.copy()
            nxt[nxt < 0] = 0
            reach = (live[nxt] & (self.trans >= 0)).any(axis=1)
            new = live | reach
            changed = bool((new != live).any())
            live = new
        return live


def nfa_to_dfa(nfa: Nfa, max_states: int = MAX_DFA_STATES, prune_dead: bool = True) -> Dfa:
    start = nfa.closure([nfa.start])
    ids = {start: 0}
    order = [start]
    rows: list[np.ndarray] = []
    i = 0
    while i < len(order):
        cur = order[i]
        i += 1
        row = np.full(256, -1, dtype=np.int32)
        by_byte: dict[int, set[int]] = {}
        for s in cur:
            for cls, tgt in nfa.trans[s]:
                for b in cls:
                    by_byte.setdefault(b, set()).add(tgt)
        memo: dict[frozenset[int], int] = {}
        for b, tg in by_byte.items():
            key = frozenset(tg)
            if key not in memo:
                cl = nfa.closure(key)
                if cl not in ids:
                    if len(order) >= max_states:
                        raise RegexError(f"automaton exceeds {max_states} states")
                    ids[cl] = len(order)
                    order.append(cl)
                memo[key] = ids[cl]
            row[b] = memo[key]
        rows.append(row)
    dfa = Dfa(np.stack(rows), np.array([nfa.accept in st for st in order], dtype=bool))
    if prune_dead:
        live = dfa.live_states()
        t = dfa.trans.copy()
        dead_target = (t >= 0) & ~live[np.where(t >= 0, t, 0)]
        t[dead_target] = -1
        dfa = Dfa(t, dfa.accepting)
    return dfa


def compile_regex(pattern: str, max_states: int = MAX_DFA_STATES) -> Dfa:
    return nfa_to_dfa(regex_to_nfa(pattern), max_states)

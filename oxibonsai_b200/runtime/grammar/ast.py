"""Grammar AST over bytes, BNF and GBNF parsers.

Reference: crates/oxibonsai-runtime/src/grammar/ast.rs:34-121 (``Symbol`` / ``Rule`` / ``Grammar``), bnf_parser.rs and
gbnf_parser.rs (the llama.cpp grammar dialect: ``name ::= "lit" [a-z] other ( a | b )* # comment``).  Terminals are
sets of bytes: a quoted literal becomes one single-byte set per byte, a character class becomes a set of ASCII bytes plus
alternatives for the UTF-8 sequences it spans.  Groups and quantifiers are desugared into fresh rules, so the recogniser
only ever sees plain context-free productions.
"""
from __future__ import annotations

from dataclasses import dataclass, field

ByteSet = frozenset


@dataclass(frozen=True)
class Term:
    """One byte out of ``bytes``."""
    bytes: ByteSet

    def __repr__(self) -> str:
        b = sorted(self.bytes)
        return f"Term({bytes(b[:8])!r}{'...' if len(b) > 8 else ''})"


@dataclass(frozen=True)
class NonTerm:
    name: str


Symbol = Term | NonTerm


@dataclass
class Rule:
    name: str
    alternatives: list[list[Symbol]] = field(default_factory=list)


class GrammarError(ValueError):
    pass


class Grammar:
    def __init__(self, start: str = "root"):
        self.start = start
        self.rules: dict[str, Rule] = {}
        self._fresh = 0

    def add(self, name: str, alternative: list[Symbol]) -> None:
        self.rules.setdefault(name, Rule(name)).alternatives.append(list(alternative))

    def fresh(self, hint: str) -> str:
        self._fresh += 1
        return f"{hint}${self._fresh}"

    def validate(self) -> "Grammar":
        if self.start not in self.rules:
            raise GrammarError(f"start rule {self.start!r} is not defined")
        for r in self.rules.values():
            for alt in r.alternatives:
                for s in alt:
                    if isinstance(s, NonTerm) and s.name not in self.rules:
                        raise GrammarError(f"rule {r.name!r} refers to undefined rule {s.name!r}")
        return self

    def nullable(self) -> set[str]:
        out: set[str] = set()
        changed = True
        while changed:
            changed = False
            for r in self.rules.values():
                if r.name in out:
                    continue
                if any(all(isinstance(s, NonTerm) and s.name in out for s in alt) for alt in r.alternatives):
                    out.add(r.name)
                    changed = True
        return out

    def first_sets(self) -> dict[str, ByteSet]:
        """Bytes that can start a derivation of each rule."""
        nullable = self.nullable()
        first: dict[str, set[int]] = {n: set() for n in self.rules}
        changed = True
        while changed:
            changed = False
            for r in self.rules.values():
                for alt in r.alternatives:
                    for s in alt:
                        add = s.bytes if isinstance(s, Term) else first[s.name]
                        if not add <= first[r.name]:
                            first[r.name] |= add
                            changed = True
                        if isinstance(s, Term) or s.name not in nullable:
                            break
        return {k: frozenset(v) for k, v in first.items()}

    # ---- helpers used by the compilers -------------------------------------------------------------------------
    def literal(self, data: bytes) -> list[Symbol]:
        return [Term(frozenset([b])) for b in data]

    def star(self, body: list[Symbol], hint: str = "rep") -> NonTerm:
        # left-recursive: an Earley chart then holds a constant number of items per repetition (the right-recursive form
        # leaves one pending item per repetition and completes all of them at every position where the body may end)
        n = self.fresh(hint)
        self.add(n, [])
        self.add(n, [NonTerm(n)] + body)
        return NonTerm(n)

    def plus(self, body: list[Symbol], hint: str = "rep") -> list[Symbol]:
        return body + [self.star(body, hint)]

    def repeat(self, body: list[Symbol], lo: int, hi: int | None, hint: str = "rep") -> list[Symbol]:
        """``body{lo,hi}`` (``hi`` None: no upper bound) in a number of rules linear in the bounds: ``lo`` copies behind a
        chain of rules of at most 64 copies each, then either ``body*`` or a chain of nested optionals
        ``opt_k ::= | body opt_(k-1)``."""
        out: list[Symbol] = []
        if lo > 0:
            copies = lo
            while copies > 0:                                   # long runs are cut into rules of bounded length
                n = min(copies, 64)
                name = self.fresh(hint + "_n")
                self.add(name, body * n)
                out.append(NonTerm(name))
                copies -= n
        if hi is None:
            out.append(self.star(body, hint))
        elif hi > lo:
            nxt: NonTerm | None = None
            for _ in range(hi - lo):
                name = self.fresh(hint + "_o")
                self.add(name, [])
                self.add(name, body + ([nxt] if nxt is not None else []))
                nxt = NonTerm(name)
            out.append(nxt)
        return out

    def optional(self, body: list[Symbol], hint: str = "opt") -> NonTerm:
        n = self.fresh(hint)
        self.add(n, [])
        self.add(n, body)
        return NonTerm(n)

    def group(self, alternatives: list[list[Symbol]], hint: str = "grp") -> NonTerm:
        n = self.fresh(hint)
        for a in alternatives:
            self.add(n, a)
        return NonTerm(n)


# ---- UTF-8 aware character classes ------------------------------------------------------------------------------------------
_CONT = frozenset(range(0x80, 0xC0))


def _any_multibyte(g: Grammar) -> NonTerm:
    """Any well-formed multi-byte UTF-8 sequence (coarse: lead byte by length, continuation bytes unconstrained)."""
    if "utf8$multi" not in g.rules:
        c = Term(_CONT)
        g.add("utf8$multi", [Term(frozenset(range(0xC2, 0xE0))), c])
        g.add("utf8$multi", [Term(frozenset(range(0xE0, 0xF0))), c, c])
        g.add("utf8$multi", [Term(frozenset(range(0xF0, 0xF5))), c, c, c])
    return NonTerm("utf8$multi")


def char_class(g: Grammar, ranges: list[tuple[int, int]], negated: bool) -> list[Symbol]:
    """Symbols matching one character of the class given as code point ranges."""
    ascii_set: set[int] = set()
    wide: list[tuple[int, int]] = []
    for lo, hi in ranges:
        ascii_set |= set(range(lo, min(hi, 127) + 1))
        if hi > 127:
            wide.append((max(lo, 128), hi))
    if negated:
        alts: list[list[Symbol]] = []
        rest = frozenset(range(128)) - ascii_set
        if rest:
            alts.append([Term(rest)])
        alts.append([_any_multibyte(g)])     # coarse: negated classes admit every non-ASCII character
        return [g.group(alts, "cls")]
    alts = []
    if ascii_set:
        alts.append([Term(frozenset(ascii_set))])
    n_wide = sum(hi - lo + 1 for lo, hi in wide)
    if n_wide > 2048:
        alts.append([_any_multibyte(g)])
    else:
        for lo, hi in wide:
            for cp in range(lo, hi + 1):
                if 0xD800 <= cp <= 0xDFFF:
                    continue
                alts.append(g.literal(chr(cp).encode("utf-8")))
    if not alts:
        raise GrammarError("empty character class")
    return alts[0] if len(alts) == 1 else [g.group(alts, "cls")]


# ---- GBNF ----------------------------------------------------------------------------------------------------------------------
class _Gbnf:
    def __init__(self, text: str, g: Grammar):
        self.s, self.i, self.g = text, 0, g

    def ws(self, newlines: bool) -> None:
        while self.i < len(self.s):
            c = self.s[self.i]
            if c == "#":
                while self.i < len(self.s) and self.s[self.i] != "\n":
                    self.i += 1
            elif c in " \t" or (newlines and c in "\r\n"):
                self.i += 1
            else:
                break

    def name(self) -> str:
        j = self.i
        while j < len(self.s) and (self.s[j].isalnum() or self.s[j] in "-_"):
            j += 1
        if j == self.i:
            raise GrammarError(f"expected a rule name at offset {self.i}")
        out, self.i = self.s[self.i:j], j
        return out

    def char(self) -> int:
        c = self.s[self.i]
        self.i += 1
        if c != "\\":
            return ord(c)
        e = self.s[self.i]
        self.i += 1
        simple = {"n": 10, "t": 9, "r": 13, "\\": 92, '"': 34, "[": 91, "]": 93, "-": 45, "^": 94, "'": 39}
        if e in simple:
            return simple[e]
        width = {"x": 2, "u": 4, "U": 8}.get(e)
        if width is None:
            raise GrammarError(f"unknown escape \\{e}")
        v = int(self.s[self.i:self.i + width], 16)
        self.i += width
        return v

    def parse(self) -> None:
        self.ws(True)
        while self.i < len(self.s):
            lhs = self.name()
            self.ws(False)
            if not self.s.startswith("::=", self.i):
                raise GrammarError(f"expected ::= after {lhs!r}")
            self.i += 3
            for alt in self.alternatives(lhs, top=True):
                self.g.add(lhs, alt)
            self.ws(True)

    def alternatives(self, hint: str, top: bool) -> list[list[Symbol]]:
        alts = [self.sequence(hint, top)]
        while self.i < len(self.s) and self.s[self.i] == "|":
            self.i += 1
            alts.append(self.sequence(hint, top))
        return alts

    def at_rule_start(self) -> bool:
        """True when the text at the cursor (after blank lines) opens a new ``name ::=`` definition."""
        j = self.i
        while j < len(self.s) and (self.s[j].isalnum() or self.s[j] in "-_"):
            j += 1
        if j == self.i:
            return False
        while j < len(self.s) and self.s[j] in " \t":
            j += 1
        return self.s.startswith("::=", j)

    def sequence(self, hint: str, top: bool) -> list[Symbol]:
        seq: list[Symbol] = []
        while True:
            self.ws(False)
            if top and self.i < len(self.s) and self.s[self.i] in "\r\n":
                # a definition may continue on the next line unless that line starts a new rule (or begins with |)
                save = self.i
                self.ws(True)
                if self.i >= len(self.s) or self.at_rule_start():
                    self.i = save
                    return seq
                continue
            if not top:
                self.ws(True)
            if self.i >= len(self.s) or self.s[self.i] in "|)":
                return seq
            item = self.item(hint)
            self.ws(False)
            if self.i < len(self.s) and self.s[self.i] in "*+?":
                q = self.s[self.i]
                self.i += 1
                item = [self.g.star(item, hint)] if q == "*" else (self.g.plus(item, hint) if q == "+" else [self.g.optional(item, hint)])
            elif self.i < len(self.s) and self.s[self.i] == "{":
                j = self.s.index("}", self.i)
                parts = self.s[self.i + 1:j].split(",")
                self.i = j + 1
                lo = int(parts[0] or 0)
                hi = lo if len(parts) == 1 else (int(parts[1]) if parts[1].strip() else None)
                body = item
                item = [s for _ in range(lo) for s in body]
                if hi is None:
                    item.append(self.g.star(body, hint))
                else:
                    for _ in range(hi - lo):
                        item.append(self.g.optional(body, hint))
            seq.extend(item)

    def item(self, hint: str) -> list[Symbol]:
        c = self.s[self.i]
        if c == '"':
            self.i += 1
            out = bytearray()
            while self.s[self.i] != '"':
                out += chr(self.char()).encode("utf-8")
            self.i += 1
            return self.g.literal(bytes(out))
        if c == "[":
            self.i += 1
            neg = self.s[self.i] == "^"
            if neg:
                self.i += 1
            ranges = []
            while self.s[self.i] != "]":
                lo = self.char()
                hi = lo
                if self.s[self.i] == "-" and self.s[self.i + 1] != "]":
                    self.i += 1
                    hi = self.char()
                ranges.append((lo, hi))
            self.i += 1
            return char_class(self.g, ranges, neg)
        if c == "(":
            self.i += 1
            alts = self.alternatives(hint, top=False)
            self.ws(True)
            if self.i >= len(self.s) or self.s[self.i] != ")":
                raise GrammarError("missing )")
            self.i += 1
            return [self.g.group(alts, hint)]
        if c == ".":
            self.i += 1
            return char_class(self.g, [(10, 10)], True)
        return [NonTerm(self.name())]


def parse_gbnf(text: str, start: str = "root") -> Grammar:
    g = Grammar(start)
    _Gbnf(text, g).parse()
    return g.validate()


def parse_bnf(text: str, start: str | None = None) -> Grammar:
    """Classic BNF: ``<expr> ::= <term> "+" <expr> | <term>``; terminals are quoted with ' or "."""
    g = Grammar(start or "")
    first = None
    for raw in text.splitlines():
        line = raw.split("#", 1)[0].strip() if not ('"#' in raw or "'#" in raw) else raw.strip()
        if not line:
            continue
        if "::=" not in line:
            raise GrammarError(f"expected ::= in {raw!r}")
        lhs, rhs = line.split("::=", 1)
        name = lhs.strip().strip("<>").strip()
        first = first or name
        i, alt, alts = 0, [], []
        while i < len(rhs):
            c = rhs[i]
            if c.isspace():
                i += 1
            elif c == "|":
                alts.append(alt)
                alt = []
                i += 1
            elif c == "<":
                j = rhs.index(">", i)
                alt.append(NonTerm(rhs[i + 1:j].strip()))
                i = j + 1
            elif c in "\"'":
                j = rhs.index(c, i + 1)
                alt.extend(g.literal(rhs[i + 1:j].encode("utf-8")))
                i = j + 1
            else:
                j = i
                while j < len(rhs) and not rhs[j].isspace() and rhs[j] not in "|<\"'":
                    j += 1
                alt.append(NonTerm(rhs[i:j]))
                i = j
        alts.append(alt)
        for a in alts:
            g.add(name, a)
    g.start = start or first or ""
    return g.validate()

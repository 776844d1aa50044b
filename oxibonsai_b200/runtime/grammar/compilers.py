"""Grammar compilers: JSON Schema -> grammar, regex -> right-linear grammar, and canned grammars.

Reference: crates/oxibonsai-runtime/src/grammar/json_schema_compiler.rs (object / array / string / number / integer /
boolean / null / enum / const / anyOf / oneOf, required and optional properties in declaration order),
regex_compiler.rs (DFA -> one rule per state) and examples.rs (JSON, arithmetic, identifier lists ...).
"""
from __future__ import annotations

import json
from typing import Any

from .ast import Grammar, GrammarError, NonTerm, Symbol, Term, parse_gbnf
from .regex_compiler import Dfa, compile_regex

JSON_GBNF = r'''
root   ::= ws value ws
value  ::= object | array | string | number | "true" | "false" | "null"
object ::= "{" ws ( member ( ws "," ws member )* )? ws "}"
member ::= string ws ":" ws value
array  ::= "[" ws ( value ( ws "," ws value )* )? ws "]"
string ::= "\"" char* "\""
char   ::= [^"\\\x00-\x1f] | "\\" ( ["\\/bfnrt] | "u" hex hex hex hex )
hex    ::= [0-9a-fA-F]
number ::= "-"? ( "0" | [1-9] [0-9]* ) ( "." [0-9]+ )? ( [eE] [-+]? [0-9]+ )?
ws     ::= [ \t\n\r]*
'''

ARITHMETIC_GBNF = r'''
root   ::= expr
expr   ::= term ( ws [-+] ws term )*
term   ::= factor ( ws [*/] ws factor )*
factor ::= number | "(" ws expr ws ")"
number ::= [0-9]+ ( "." [0-9]+ )?
ws     ::= [ ]*
'''

IDENT_LIST_GBNF = r'''
root  ::= ident ( "," " "? ident )*
ident ::= [a-zA-Z_] [a-zA-Z0-9_]*
'''

YES_NO_GBNF = 'root ::= "yes" | "no"\n'


def json_grammar() -> Grammar:
    return parse_gbnf(JSON_GBNF)


def arithmetic_grammar() -> Grammar:
    return parse_gbnf(ARITHMETIC_GBNF)


def identifier_list_grammar() -> Grammar:
    return parse_gbnf(IDENT_LIST_GBNF)


def yes_no_grammar() -> Grammar:
    return parse_gbnf(YES_NO_GBNF)


def regex_to_grammar(pattern: str, start: str = "root") -> Grammar:
    """One rule per DFA state: ``S_i ::= byte-class S_j | ... | (empty when accepting)``."""
    dfa: Dfa = compile_regex(pattern)
    g = Grammar(start)
    name = lambda s: start if s == 0 else f"{start}$s{s}"
    for s in range(dfa.n_states):
        by_target: dict[int, set[int]] = {}
        for b in range(256):
            t = int(dfa.trans[s, b])
            if t >= 0:
                by_target.setdefault(t, set()).add(b)
        for t, bs in by_target.items():
            g.add(name(s), [Term(frozenset(bs)), NonTerm(name(t))])
        if dfa.accepting[s]:
            g.add(name(s), [])
        if name(s) not in g.rules:
            g.add(name(s), [Term(frozenset())])     # dead state: no byte matches
    return g.validate()


class _SchemaCompiler:
    def __init__(self):
        self.g = parse_gbnf(JSON_GBNF)
        self.g.start = "schema$root"
        self.n = 0

    def lit(self, s: str) -> list[Symbol]:
        return self.g.literal(s.encode("utf-8"))

    def ws(self) -> Symbol:
        return NonTerm("ws")

    def new(self, hint: str) -> str:
        self.n += 1
        return f"schema${hint}{self.n}"

    def compile(self, schema: Any) -> Grammar:
        v = self.value(schema)
        self.g.add("schema$root", [self.ws(), v, self.ws()])
        return self.g.validate()

    def value(self, sc: Any) -> Symbol:
        if sc is True or sc == {}:
            return NonTerm("value")
        if not isinstance(sc, dict):
            raise GrammarError(f"unsupported schema node {sc!r}")
        if "const" in sc:
            return self.g.group([self.lit(json.dumps(sc["const"], separators=(",", ":"), ensure_ascii=False))], "const")
        if "enum" in sc:
            return self.g.group([self.lit(json.dumps(v, separators=(",", ":"), ensure_ascii=False)) for v in sc["enum"]], "enum")
        for key in ("anyOf", "oneOf"):
            if key in sc:
                return self.g.group([[self.value(s)] for s in sc[key]], key)
        t = sc.get("type")
        if isinstance(t, list):
            return self.g.group([[self.value({**sc, "type": x})] for x in t], "types")
        if t == "object" or (t is None and "properties" in sc):
            return self.obj(sc)
        if t == "array":
            return self.arr(sc)
        if t == "string":
            return self.string(sc)
        if t == "integer":
            name = self.new("int")
            self.g.add(name, parse_int_body(self.g))
            return NonTerm(name)
        if t == "number":
            return NonTerm("number")
        if t == "boolean":
            return self.g.group([self.lit("true"), self.lit("false")], "bool")
        if t == "null":
            return self.g.group([self.lit("null")], "null")
        if t is None:
            return NonTerm("value")
        raise GrammarError(f"unsupported schema type {t!r}")

    def string(self, sc: dict) -> Symbol:
        if "pattern" in sc:
            inner = regex_to_grammar(sc["pattern"], self.new("pat"))
            self.g.rules.update(inner.rules)
            return self.g.group([self.lit('"') + [NonTerm(inner.start)] + self.lit('"')], "patstr")
        lo, hi = sc.get("minLength"), sc.get("maxLength")
        if lo is None and hi is None:
            return NonTerm("string")
        lo = int(lo or 0)
        if hi is not None and int(hi) < lo:
            raise GrammarError(f"maxLength {hi} is below minLength {lo}")
        body = self.g.repeat([NonTerm("char")], lo, None if hi is None else int(hi), "chars")
        return self.g.group([self.lit('"') + body + self.lit('"')], "lenstr")

    def arr(self, sc: dict) -> Symbol:
        item = self.value(sc.get("items", True))
        lo, hi = int(sc.get("minItems", 0)), sc.get("maxItems")
        sep: list[Symbol] = [self.ws()] + self.lit(",") + [self.ws()]
        more: list[Symbol] = sep + [item]
        name = self.new("arr")
        if hi is not None and int(hi) < lo:
            raise GrammarError(f"maxItems {hi} is below minItems {lo}")
        if lo == 0:
            self.g.add(name, self.lit("[") + [self.ws()] + self.lit("]"))
        if hi is None or int(hi) >= 1:
            # the first item, then (", " item){lo-1, hi-1}: rules linear in the bounds
            rest = self.g.repeat(more, max(lo - 1, 0), None if hi is None else int(hi) - 1, "items")
            self.g.add(name, self.lit("[") + [self.ws(), item] + rest + [self.ws()] + self.lit("]"))
        return NonTerm(name)

    def obj(self, sc: dict) -> Symbol:
        props: dict = sc.get("properties", {})
        required = set(sc.get("required", []))
        name = self.new("obj")
        if not props:
            return NonTerm("object")
        members = []
        for key, sub in props.items():
            m = self.lit(json.dumps(key, ensure_ascii=False)) + [self.ws()] + self.lit(":") + [self.ws(), self.value(sub)]
            members.append((key in required, m))
        sep: list[Symbol] = [self.ws()] + self.lit(",") + [self.ws()]
        # properties appear in declaration order; optional ones may be skipped.  state = (next property, "has a member been
        # emitted yet"): one rule per state, so the grammar is linear in the number of properties however many are optional
        states: dict[tuple[int, bool], Symbol] = {}

        def chain(i: int, emitted: bool) -> Symbol:
            if (i, emitted) in states:
                return states[(i, emitted)]
            nm = self.new("mem")
            states[(i, emitted)] = NonTerm(nm)
            if i == len(members):
                self.g.add(nm, [])
                return NonTerm(nm)
            req, m = members[i]
            with_sep = (sep if emitted else []) + m + [chain(i + 1, True)]
            self.g.add(nm, with_sep)
            if not req:
                self.g.add(nm, [chain(i + 1, emitted)])
            return NonTerm(nm)
        self.g.add(name, self.lit("{") + [self.ws(), chain(0, False), self.ws()] + self.lit("}"))
        return NonTerm(name)


def parse_int_body(g: Grammar) -> list[Symbol]:
    digits = g.star([Term(frozenset(range(48, 58)))], "digits")
    nz = g.group([[Term(frozenset([48]))], [Term(frozenset(range(49, 58))), digits]], "intbody")
    return [g.optional([Term(frozenset([45]))], "sign"), nz]


def json_schema_to_grammar(schema: Any) -> Grammar:
    if isinstance(schema, str):
        schema = json.loads(schema)
    return _SchemaCompiler().compile(schema)

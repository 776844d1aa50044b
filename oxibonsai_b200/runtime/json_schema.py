"""JSON Schema subset: parser, validator, incremental prefix checker, template and example generators.

Reference: crates/oxibonsai-runtime/src/json_schema.rs:24-1117 (``SchemaType`` with object / array / string / number /
integer / boolean / null / enum / any-of, ``parse_schema``, ``SchemaState::feed_char`` / ``valid_next_chars``,
``validate_against_schema``, ``schema_template``, ``schema_example``).  The incremental checker here is the grammar
engine compiled from the schema, so "which characters may follow" is exact rather than heuristic.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Any


class SchemaError(ValueError):
    pass


_TYPES = ("object", "array", "string", "number", "integer", "boolean", "null")


@dataclass
class Schema:
    type: str | None = None                       # one of _TYPES, "enum", "any_of", "const" or None (anything)
    properties: dict[str, "Schema"] = field(default_factory=dict)
    required: list[str] = field(default_factory=list)
    items: "Schema | None" = None
    enum: list[Any] | None = None
    const: Any = None
    any_of: list["Schema"] = field(default_factory=list)
    minimum: float | None = None
    maximum: float | None = None
    min_length: int | None = None
    max_length: int | None = None
    min_items: int | None = None
    max_items: int | None = None
    pattern: str | None = None
    additional_properties: bool = True
    raw: Any = None

    def type_name(self) -> str:
        return self.type or "any"

    def is_required_property(self, key: str) -> bool:
        return key in self.required


def parse_schema(schema: str | dict | bool) -> Schema:
    if isinstance(schema, str):
        try:
            schema = json.loads(schema)
        except json.JSONDecodeError as e:
            raise SchemaError(f"schema is not valid JSON: {e}") from None
    if schema is True or schema == {}:
        return Schema(raw=schema)
    if not isinstance(schema, dict):
        raise SchemaError(f"unsupported schema node {schema!r}")
    s = Schema(raw=schema)
    if "const" in schema:
        s.type, s.const = "const", schema["const"]
        return s
    if "enum" in schema:
        if not isinstance(schema["enum"], list) or not schema["enum"]:
            raise SchemaError("enum must be a non-empty list")
        s.type, s.enum = "enum", list(schema["enum"])
        return s
    for key in ("anyOf", "oneOf"):
        if key in schema:
            s.type, s.any_of = "any_of", [parse_schema(x) for x in schema[key]]
            return s
    t = schema.get("type")
    if isinstance(t, list):
        s.type, s.any_of = "any_of", [parse_schema({**schema, "type": x}) for x in t]
        return s
    if t is None and "properties" in schema:
        t = "object"
    if t is not None and t not in _TYPES:
        raise SchemaError(f"unknown type {t!r}")
    s.type = t
    if t == "object":
        s.properties = {k: parse_schema(v) for k, v in schema.get("properties", {}).items()}
        s.required = list(schema.get("required", []))
        for r in s.required:
            if r not in s.properties:
                raise SchemaError(f"required property {r!r} is not declared")
        s.additional_properties = bool(schema.get("additionalProperties", True))
    elif t == "array":
        s.items = parse_schema(schema["items"]) if "items" in schema else None
        s.min_items, s.max_items = schema.get("minItems"), schema.get("maxItems")
    elif t == "string":
        s.min_length, s.max_length, s.pattern = schema.get("minLength"), schema.get("maxLength"), schema.get("pattern")
    elif t in ("number", "integer"):
        s.minimum, s.maximum = schema.get("minimum"), schema.get("maximum")
    return s


def _check(v: Any, s: Schema, path: str, errs: list[str]) -> None:
    t = s.type
    if t is None:
        return
    if t == "const":
        if v != s.const:
            errs.append(f"{path}: expected {s.const!r}")
    elif t == "enum":
        if v not in s.enum:
            errs.append(f"{path}: {v!r} is not one of {s.enum!r}")
    elif t == "any_of":
        if not any(not validate_value(v, a) for a in s.any_of):
            errs.append(f"{path}: matches none of the alternatives")
    elif t == "object":
        if not isinstance(v, dict):
            errs.append(f"{path}: expected an object")
            return
        for r in s.required:
            if r not in v:
                errs.append(f"{path}: missing required property {r!r}")
        for k, x in v.items():
            if k in s.properties:
                _check(x, s.properties[k], f"{path}.{k}", errs)
            elif not s.additional_properties:
                errs.append(f"{path}: unexpected property {k!r}")
    elif t == "array":
        if not isinstance(v, list):
            errs.append(f"{path}: expected an array")
            return
        if s.min_items is not None and len(v) < s.min_items:
            errs.append(f"{path}: fewer than {s.min_items} items")
        if s.max_items is not None and len(v) > s.max_items:
            errs.append(f"{path}: more than {s.max_items} items")
        if s.items is not None:
            for i, x in enumerate(v):
                _check(x, s.items, f"{path}[{i}]", errs)
    elif t == "string":
        if not isinstance(v, str):
            errs.append(f"{path}: expected a string")
            return
        if s.min_length is not None and len(v) < s.min_length:
            errs.append(f"{path}: shorter than {s.min_length}")
        if s.max_length is not None and len(v) > s.max_length:
            errs.append(f"{path}: longer than {s.max_length}")
        if s.pattern is not None and re.fullmatch(s.pattern, v) is None:
            errs.append(f"{path}: does not match {s.pattern!r}")
    elif t in ("number", "integer"):
        if isinstance(v, bool) or not isinstance(v, (int, float)) or (t == "integer" and not float(v).is_integer()):
            errs.append(f"{path}: expected {'an integer' if t == 'integer' else 'a number'}")
            return
        if s.minimum is not None and v < s.minimum:
            errs.append(f"{path}: below {s.minimum}")
        if s.maximum is not None and v > s.maximum:
            errs.append(f"{path}: above {s.maximum}")
    elif t == "boolean":
        if not isinstance(v, bool):
            errs.append(f"{path}: expected a boolean")
    elif t == "null":
        if v is not None:
            errs.append(f"{path}: expected null")


def validate_value(value: Any, schema: Schema) -> list[str]:
    errs: list[str] = []
    _check(value, schema, "$", errs)
    return errs


def validate_against_schema(text: str, schema: Schema | str | dict) -> bool:
    s = schema if isinstance(schema, Schema) else parse_schema(schema)
    try:
        v = json.loads(text)
    except json.JSONDecodeError:
        return False
    return not validate_value(v, s)


class SchemaState:
    """Incremental checker: feed characters, ask what may follow, ask whether the text is a complete instance."""

    def __init__(self, schema: Schema | str | dict):
        from .grammar.compilers import json_schema_to_grammar
        from .grammar.earley import EarleyRecognizer
        s = schema if isinstance(schema, Schema) else parse_schema(schema)
        self.schema = s
        self._rec = EarleyRecognizer(json_schema_to_grammar(s.raw if s.raw is not None else True))
        self._buf: list[str] = []

    def feed_char(self, ch: str) -> bool:
        ok = self._rec.feed_bytes(ch.encode("utf-8"))
        if ok:
            self._buf.append(ch)
        return ok

    def feed(self, text: str) -> bool:
        return all(self.feed_char(c) for c in text)

    def valid_next_chars(self) -> list[str]:
        return [chr(b) for b in sorted(self._rec.next_bytes()) if b < 128]

    def is_complete(self) -> bool:
        return self._rec.is_complete()

    def buffer(self) -> str:
        return "".join(self._buf)

    def depth(self) -> int:
        d, in_str, esc = 0, False, False
        for c in self._buf:
            if in_str:
                esc = (c == "\\") and not esc
                if c == '"' and not esc:
                    in_str = False
            elif c == '"':
                in_str = True
            elif c in "{[":
                d += 1
            elif c in "}]":
                d -= 1
        return d


def schema_template(schema: Schema | str | dict) -> str:
    """A skeleton with placeholders, e.g. ``{"name": <string>, "age": <integer>}``."""
    s = schema if isinstance(schema, Schema) else parse_schema(schema)
    t = s.type
    if t == "object":
        return "{" + ", ".join(f"{json.dumps(k)}: {schema_template(v)}" for k, v in s.properties.items()) + "}"
    if t == "array":
        return "[" + (schema_template(s.items) if s.items else "<any>") + ", ...]"
    if t == "enum":
        return "<" + " | ".join(json.dumps(v) for v in s.enum) + ">"
    if t == "const":
        return json.dumps(s.const)
    if t == "any_of":
        return "<" + " | ".join(schema_template(a) for a in s.any_of) + ">"
    return f"<{t or 'any'}>"


def schema_example(schema: Schema | str | dict) -> Any:
    """A minimal value that validates."""
    s = schema if isinstance(schema, Schema) else parse_schema(schema)
    t = s.type
    if t == "object":
        return {k: schema_example(v) for k, v in s.properties.items() if k in s.required or len(s.properties) <= 8}
    if t == "array":
        n = max(s.min_items or 0, 1 if s.items else 0)
        return [schema_example(s.items) if s.items else None for _ in range(n)]
    if t == "string":
        return "x" * max(s.min_length or 0, 0) if not s.pattern else _pattern_example(s.pattern)
    if t == "integer":
        lo = int(s.minimum) if s.minimum is not None else 0
        return lo if s.maximum is None or lo <= s.maximum else int(s.maximum)
    if t == "number":
        return float(s.minimum) if s.minimum is not None else 0.0
    if t == "boolean":
        return True
    if t == "enum":
        return s.enum[0]
    if t == "const":
        return s.const
    if t == "any_of":
        return schema_example(s.any_of[0])
    return None


def _pattern_example(pattern: str) -> str:
    """Shortest string of a regular expression (breadth-first walk of its DFA)."""
    from .grammar.regex_compiler import compile_regex
    dfa = compile_regex(pattern)
    seen, frontier = {0: b""}, [0]
    while frontier:
        nxt = []
        for st in frontier:
            if dfa.accepting[st]:
                return seen[st].decode("utf-8", errors="replace")
            for b in dfa.next_bytes(st):
                t = int(dfa.trans[st, b])
                if t not in seen:
                    seen[t] = seen[st] + bytes([int(b)])
                    nxt.append(t)
        frontier = nxt
    return ""

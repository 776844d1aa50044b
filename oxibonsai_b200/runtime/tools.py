"""Function / tool calling: definitions, the system prompt that lists them, parsing and validation of the model's calls,
and a grammar that forces the output to be a well-formed call of one of the tools.

Reference: crates/oxibonsai-runtime/src/tool_calling.rs - error kinds (:23-52), ``new_tool_call_id`` / ``make_tool_call``
(:60-85), ``select_tool`` (parse, check the name against the tool list, check that the arguments are JSON; :96-133),
``build_tool_constraint`` (one alternative per tool: ``<tool_call>{"name":"X","arguments":`` + the tool's parameter schema
compiled to a grammar + ``}</tool_call>``; :145-235), ``ToolRegistry`` (:246-280) and ``validate_tool_arguments`` (object +
required fields; :289-325); request / response shapes in api_types.rs:13-345.  Here the constraint is a
:class:`~oxibonsai_b200.runtime.constrained.GrammarConstraint`, so with ``tool_choice`` set the GPU sampler can only emit
tokens that keep the output a valid call.
"""
from __future__ import annotations

import json
import re
import uuid
from typing import Any, Iterable


class ToolCallError(ValueError):
    """Base of the tool-calling errors; ``kind`` is the reference's variant name."""
    kind = "ToolCallError"


class NoToolCallFound(ToolCallError):
    kind = "NoToolCallFound"

    def __init__(self):
        super().__init__("no tool call found in model output")


class UnknownTool(ToolCallError):
    kind = "UnknownTool"

    def __init__(self, name: str):
        super().__init__(f"unknown tool: '{name}'")
        self.name = name


class MalformedArguments(ToolCallError):
    kind = "MalformedArguments"

    def __init__(self, reason: str):
        super().__init__(f"malformed tool arguments: {reason}")
        self.reason = reason


class GrammarCompileError(ToolCallError):
    kind = "GrammarCompileError"

    def __init__(self, reason: str):
        super().__init__(f"grammar compile error: {reason}")
        self.reason = reason


class EmptyToolList(ToolCallError):
    kind = "EmptyToolList"

    def __init__(self):
        super().__init__("tool list is empty")


def _function(tool: dict) -> dict:
    """The ``function`` object of an OpenAI tool definition (a bare function object is accepted as well)."""
    fn = tool.get("function", tool) if isinstance(tool, dict) else None
    if not isinstance(fn, dict) or not isinstance(fn.get("name"), str) or not fn["name"]:
        raise ToolCallError("a tool definition needs a function name")
    return fn


def new_tool_call_id() -> str:
    return "call_" + uuid.uuid4().hex[:24]


def make_tool_call(call_id: str, name: str, arguments: str | dict) -> dict:
    """The OpenAI ``tool_calls`` entry; ``arguments`` is kept as the JSON text the model wrote."""
    return {"id": call_id, "type": "function",
            "function": {"name": name, "arguments": arguments if isinstance(arguments, str) else json.dumps(arguments)}}


def tools_system_prompt(tools: list[dict]) -> str:
    lines = ["You can call the following tools. To call one, answer with a JSON object",
             '{"name": <tool name>, "arguments": {...}} and nothing else.', ""]
    for t in tools:
        fn = t.get("function", t)
        lines.append(f"- {fn.get('name')}: {fn.get('description', '')}")
        if fn.get("parameters"):
            lines.append(f"  parameters: {json.dumps(fn['parameters'], sort_keys=True)}")
    return "\n".join(lines)


def _json_objects(text: str):
    depth, start, in_str, esc = 0, None, False, False
    for i, ch in enumerate(text):
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
            continue
        if ch == '"':
            in_str = True
        elif ch == "{":
            if depth == 0:
                start = i
            depth += 1
        elif ch == "}" and depth:
            depth -= 1
            if depth == 0 and start is not None:
                yield text[start:i + 1]


def parse_tool_calls(text: str) -> list[dict]:
    """Extracts ``{"name": ..., "arguments": {...}}`` objects (also inside ``<tool_call>`` tags) from model output."""
    calls = []
    body = "\n".join(re.findall(r"<tool_call>(.*?)</tool_call>", text, flags=re.S)) or text
    for blob in _json_objects(body):
        try:
            obj = json.loads(blob)
        except json.JSONDecodeError:
            continue
        if isinstance(obj, dict) and isinstance(obj.get("name"), str) and isinstance(obj.get("arguments", {}), (dict, str)):
            calls.append(make_tool_call(new_tool_call_id(), obj["name"], obj.get("arguments", {})))
    return calls


class ToolRegistry:
    """Tool definitions by function name."""

    def __init__(self, tools: Iterable[dict]):
        self._map = {_function(t)["name"]: t for t in tools}

    def get(self, name: str) -> dict | None:
        return self._map.get(name)

    def names(self) -> list[str]:
        return list(self._map)

    def __len__(self) -> int:
        return len(self._map)

    def __contains__(self, name: str) -> bool:
        return name in self._map

    def is_empty(self) -> bool:
        return not self._map


def select_tool(output: str, tools: list[dict]) -> dict:
    """The first tool call in ``output``.  Raises :class:`NoToolCallFound`, :class:`UnknownTool` (when ``tools`` is not empty
    and does not define the called name) or :class:`MalformedArguments` (the arguments are not JSON)."""
    calls = parse_tool_calls(output)
    if not calls:
        raise NoToolCallFound()
    call = calls[0]
    if tools and call["function"]["name"] not in ToolRegistry(tools):
        raise UnknownTool(call["function"]["name"])
    try:
        json.loads(call["function"]["arguments"])
    except json.JSONDecodeError as e:
        raise MalformedArguments(str(e)) from e
    return call


def validate_tool_arguments(arguments: str, tool: dict, strict: bool = False) -> dict:
    """Parses the argument text of a call: it must be a JSON object holding every ``required`` property of the tool's
    parameter schema.  ``strict`` checks the whole schema (types, enums, bounds) as well."""
    try:
        parsed = json.loads(arguments)
    except json.JSONDecodeError as e:
        raise MalformedArguments(str(e)) from e
    if not isinstance(parsed, dict):
        raise MalformedArguments("tool arguments must be a JSON object")
    params = _function(tool).get("parameters") or {}
    for name in params.get("required") or []:
        if isinstance(name, str) and name not in parsed:
            raise MalformedArguments(f"missing required field '{name}'")
    if strict and params:
        from .json_schema import SchemaError, parse_schema, validate_value
        try:
            errs = validate_value(parsed, parse_schema(params))
        except SchemaError as e:
            raise MalformedArguments(str(e)) from e
        if errs:
            raise MalformedArguments("; ".join(errs[:3]))
    return parsed


def build_tool_grammar(tools: list[dict], names: Iterable[str] | None = None):
    """A grammar whose sentences are exactly ``<tool_call>{"name":"<tool>","arguments":<arguments>}</tool_call>`` for one of
    ``tools`` (restricted to ``names`` when given), the arguments following that tool's parameter schema."""
    from .grammar.ast import Grammar, NonTerm, Term
    from .grammar.compilers import json_schema_to_grammar
    if not tools:
        raise EmptyToolList()
    wanted = None if names is None else set(names)
    g = Grammar("root")
    literal = lambda text: [Term(frozenset([b])) for b in text.encode("utf-8")]
    used = 0
    for i, tool in enumerate(tools):
        fn = _function(tool)
        if wanted is not None and fn["name"] not in wanted:
            continue
        try:
            sub = json_schema_to_grammar(fn.get("parameters") or {"type": "object"}).validate()
        except Exception as e:  # noqa: BLE001 - whatever the schema compiler objects to
            raise GrammarCompileError(f"tool '{fn['name']}': {e}") from e
        # the tool's rules under names of their own
        rename = lambda n, i=i: f"t{i}.{n}"
        for rule in sub.rules.values():
            for alt in rule.alternatives:
                g.add(rename(rule.name), [NonTerm(rename(s.name)) if isinstance(s, NonTerm) else s for s in alt])
        g.add("root", literal('<tool_call>{"name":' + json.dumps(fn["name"]) + ',"arguments":') + [NonTerm(rename(sub.start))] + literal("}</tool_call>"))
        used += 1
    if not used:
        raise UnknownTool(", ".join(sorted(wanted or [])))
    return g.validate()


def build_tool_constraint(table, tools: list[dict], names: Iterable[str] | None = None, eos_token: int | None = None):
    """The token constraint of :func:`build_tool_grammar` over the vocabulary ``table``."""
    from .constrained import GrammarConstraint
    return GrammarConstraint(table, build_tool_grammar(tools, names), eos_token)


def tool_choice_names(tool_choice: Any, tools: list[dict]) -> list[str] | None:
    """Which tools a request's ``tool_choice`` forces: None = free text allowed ("auto", "none", absent), a list of names =
    the output must be a call of one of them ("required": any tool; a function object: that tool)."""
    if tool_choice in (None, "auto", "none"):
        return None
    if tool_choice == "required":
        return [_function(t)["name"] for t in tools]
    if isinstance(tool_choice, dict):
        name = (tool_choice.get("function") or {}).get("name") or tool_choice.get("name")
        if not isinstance(name, str):
            raise ToolCallError("tool_choice needs a function name")
        if name not in ToolRegistry(tools):
            raise UnknownTool(name)
        return [name]
    raise ToolCallError(f"unsupported tool_choice: {tool_choice!r}")

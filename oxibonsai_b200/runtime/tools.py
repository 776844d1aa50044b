"""Function / tool calling helpers for the chat endpoint.

Reference: tool definitions, a system prompt that lists them and a parser that recognises JSON tool invocations in the
model output (crates/oxibonsai-runtime/src/tool_calling.rs:23-289, api_extensions.rs:25-438).
"""
from __future__ import annotations

import json
import re
import uuid


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
            args = obj.get("arguments", {})
            calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                          "function": {"name": obj["name"], "arguments": args if isinstance(args, str) else json.dumps(args)}})
    return calls

"""Tool protocol: definitions, tool choice, the canonical call envelope and its JSON-Schema grammar.

The engine never executes tools (reference: crates/sllm-frontend/src/tool_protocol.rs:1-9); it constrains the
model to emit `{"tool_calls":[{"name":..., "arguments":{...}}]}` (or plain text when allowed) and parses the
result.  Bounds follow :18-30.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Optional

MAX_TOOLS = 32
MAX_TOOL_NAME = 64
MAX_TOOL_DESCRIPTION = 4096
MAX_TOOL_SCHEMA_BYTES = 64 * 1024
MAX_TOOL_CALLS = 8
_NAME = re.compile(r"^[A-Za-z0-9_-]{1,64}$")


class ToolProtocolError(ValueError):
    pass


@dataclass
class ToolDefinition:
    name: str
    description: str = ""
    parameters: dict = field(default_factory=lambda: {"type": "object", "properties": {}, "additionalProperties": False})

    def __post_init__(self):
        if not _NAME.match(self.name or ""):
            raise ToolProtocolError("tool name must match [A-Za-z0-9_-]{1,64}")
        if len(self.description.encode()) > MAX_TOOL_DESCRIPTION:
            raise ToolProtocolError("tool description too long")
        if not isinstance(self.parameters, dict) or self.parameters.get("type") != "object":
            raise ToolProtocolError("tool parameters must be an object schema")
        if len(json.dumps(self.parameters).encode()) > MAX_TOOL_SCHEMA_BYTES:
            raise ToolProtocolError("tool schema too large")


@dataclass
class ToolChoice:
    mode: str = "auto"            # none | auto | required | named
    name: Optional[str] = None


@dataclass
class ToolCall:
    id: str
    name: str
    arguments: dict


def parse_tools(raw) -> list:
    if not isinstance(raw, list) or not raw:
        raise ToolProtocolError("tools must be a non-empty array")
    if len(raw) > MAX_TOOLS:
        raise ToolProtocolError("too many tools")
    out, seen = [], set()
    for t in raw:
        if not isinstance(t, dict) or set(t) - {"type", "function"} or t.get("type") != "function":
            raise ToolProtocolError("tool entries must be {type:'function', function:{...}}")
        f = t.get("function")
        if not isinstance(f, dict) or set(f) - {"name", "description", "parameters", "strict"}:
            raise ToolProtocolError("unknown member in function definition")
        d = ToolDefinition(f.get("name"), f.get("description", "") or "", f.get("parameters") or
                           {"type": "object", "properties": {}, "additionalProperties": False})
        if d.name in seen:
            raise ToolProtocolError("duplicate tool name")
        seen.add(d.name)
        out.append(d)
    return out


def parse_tool_choice(raw, tools: list) -> ToolChoice:
    if raw is None:
        return ToolChoice("auto")
    if isinstance(raw, str):
        if raw not in ("none", "auto", "required"):
            raise ToolProtocolError("tool_choice must be none, auto, required or a named function")
        return ToolChoice(raw)
    if isinstance(raw, dict) and raw.get("type") == "function" and isinstance(raw.get("function"), dict):
        name = raw["function"].get("name")
        if name not in {t.name for t in tools}:
            raise ToolProtocolError("tool_choice names an unknown tool")
        return ToolChoice("named", name)
    raise ToolProtocolError("invalid tool_choice")


def envelope_schema(tools: list, choice: ToolChoice) -> dict:
    """JSON Schema of the canonical envelope for the grammar compiler."""
    chosen = [t for t in tools if choice.mode != "named" or t.name == choice.name]
    variants = [{"type": "object", "properties": {"name": {"const": t.name}, "arguments": t.parameters},
                 "required": ["name", "arguments"], "additionalProperties": False} for t in chosen]
    return {"type": "object", "properties": {"tool_calls": {"type": "array", "items": {"anyOf": variants}}},
            "required": ["tool_calls"], "additionalProperties": False}


def render_tool_preamble(tools: list) -> str:
    """System-prompt section that advertises the tools (deterministic ordering)."""
    lines = ["# Tools", "", "You may call one or more functions. Respond with a JSON object "
             '{"tool_calls":[{"name":<function-name>,"arguments":<args-json-object>}]}.', "", "<tools>"]
    for t in tools:
        lines.append(json.dumps({"type": "function", "function": {"name": t.name, "description": t.description,
                                                                    "parameters": t.parameters}}, sort_keys=True))
    lines.append("</tools>")
    return "\n".join(lines)


def parse_tool_calls(text: str, tools: list, id_prefix: str = "call") -> list:
    """Parses generated text into tool calls; raises when the envelope is malformed."""
    try:
        obj = json.loads(text)
    except json.JSONDecodeError as exc:
        raise ToolProtocolError(f"tool call output is not JSON: {exc.msg}") from None
    if not isinstance(obj, dict) or set(obj) != {"tool_calls"} or not isinstance(obj["tool_calls"], list):
        raise ToolProtocolError("tool call envelope must be {tool_calls:[...]}")
    if not 1 <= len(obj["tool_calls"]) <= MAX_TOOL_CALLS:
        raise ToolProtocolError("tool call count out of range")
    names = {t.name for t in tools}
    out = []
    for i, c in enumerate(obj["tool_calls"]):
        if not isinstance(c, dict) or set(c) != {"name", "arguments"} or c["name"] not in names \
                or not isinstance(c["arguments"], dict):
            raise ToolProtocolError("malformed tool call")
        out.append(ToolCall(f"{id_prefix}_{i}", c["name"], c["arguments"]))
    return out


def render_tool_result(call_id: str, content: str) -> str:
    return f"<tool_response id=\"{call_id}\">\n{content}\n</tool_response>"

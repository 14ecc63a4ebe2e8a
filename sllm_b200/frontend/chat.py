"""Chat rendering: the fixed ChatML / Qwen3.5 renderer and the sandboxed generic template provider.

Fixed renderer rules (reference: crates/sllm-frontend/src/chat.rs:26-31,850-900): every message is
`<|im_start|>{role}\n{content}<|im_end|>\n` with Qwen-style trimming; an assistant message before the last
user turn contributes only its visible answer, one after it is rendered as `<think>\n{reasoning}\n</think>\n\n
{answer}`; reasoning comes from `reasoning_content` when given, else from a leading `<think>..</think>` block of
the content; the generation prompt is `<|im_start|>assistant\n<think>\n` (thinking) or
`<|im_start|>assistant\n<think>\n\n</think>\n\n` (disabled).  Output is capped at 16 MiB.

Generic templates (reference: template.rs:19-27) run in a Jinja2 sandbox: no loader / include / import,
JSON-only context, source <= 64 KiB, output <= 16 MiB, a bounded number of render steps.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from typing import Optional

IM_START, IM_END_LINE = "<|im_start|>", "<|im_end|>\n"
GEN_THINKING = "<|im_start|>assistant\n<think>\n"
GEN_DISABLED = "<|im_start|>assistant\n<think>\n\n</think>\n\n"
MAX_RENDER_BYTES = 16 * 1024 * 1024
MAX_MESSAGES = 1024
MAX_TEMPLATE_SOURCE = 64 * 1024
TEMPLATE_FUEL = 1_000_000


class ChatRenderError(ValueError):
    pass


@dataclass
class ChatMessage:
    role: str                 # system | user | assistant
    content: str
    reasoning_content: Optional[str] = None


def _trim(s: str) -> str:
    return s.strip()


def split_reasoning(content: str, explicit: Optional[str]):
    """(reasoning, answer) of an assistant message."""
    if explicit is not None:
        return _trim(explicit), _trim(content)
    if "</think>" in content:
        head, _, tail = content.rpartition("</think>")
        reasoning = head.split("<think>")[-1] if "<think>" in head else head
        return _trim(reasoning), _trim(tail)
    return "", _trim(content)


def validate_messages(messages: list) -> None:
    if not messages:
        raise ChatRenderError("messages must not be empty")
    if len(messages) > MAX_MESSAGES:
        raise ChatRenderError("too many messages")
    seen_system = 0
    for i, m in enumerate(messages):
        if m.role not in ("system", "user", "assistant"):
            raise ChatRenderError(f"unsupported role {m.role!r}")
        if m.role == "system":
            seen_system += 1
            if i != 0:
                raise ChatRenderError("the system message must be first")
        if m.reasoning_content is not None and m.role != "assistant":
            raise ChatRenderError("reasoning_content is only valid on assistant messages")
    if seen_system > 1:
        raise ChatRenderError("at most one system message")
    if not any(m.role == "user" for m in messages):
        raise ChatRenderError("at least one user message is required")


def render_chatml(messages: list, thinking: str = "disabled", add_generation_prompt: bool = True,
                  assistant_prefill: str = "") -> str:
    """thinking: 'enabled' | 'disabled' | 'template_default' (= disabled for this renderer)."""
    validate_messages(messages)
    last_user = max(i for i, m in enumerate(messages) if m.role == "user")
    out = []
    total = 0

    def emit(s: str):
        nonlocal total
        total += len(s.encode("utf-8"))
        if total > MAX_RENDER_BYTES:
            raise ChatRenderError("rendered prompt exceeds 16 MiB")
        out.append(s)

    for i, m in enumerate(messages):
        emit(IM_START)
        if m.role in ("system", "user"):
            emit(m.role + "\n")
            emit(_trim(m.content))
        else:
            emit("assistant\n")
            reasoning, answer = split_reasoning(m.content, m.reasoning_content)
            if i < last_user:
                emit(answer)
            else:
                emit("<think>\n")
                emit(reasoning)
                emit("\n</think>\n\n")
                emit(answer)
        emit(IM_END_LINE)
    if add_generation_prompt:
        emit(GEN_THINKING if thinking == "enabled" else GEN_DISABLED)
        emit(assistant_prefill)
    return "".join(out)


RENDERER_IDENTITY = "chatml-qwen35-v1:" + hashlib.sha256((GEN_THINKING + GEN_DISABLED + IM_START + IM_END_LINE).encode()).hexdigest()[:16]


class GenericTemplate:
    """A client-supplied chat template rendered in a sandbox with hard limits."""

    def __init__(self, source: str, expected_sha256: Optional[str] = None):
        if len(source.encode("utf-8")) > MAX_TEMPLATE_SOURCE:
            raise ChatRenderError("template source exceeds 64 KiB")
        self.digest = hashlib.sha256(source.encode("utf-8")).hexdigest()
        if expected_sha256 is not None and expected_sha256.lower() != self.digest:
            raise ChatRenderError("template digest mismatch")
        for banned in ("{% include", "{% import", "{% from", "{% extends", "{%- include", "{%- import", "{%- from",
                       "{%- extends"):
            if banned in source:
                raise ChatRenderError("include / import / extends are not available in templates")
        from jinja2.sandbox import ImmutableSandboxedEnvironment
        self.env = ImmutableSandboxedEnvironment(autoescape=False, loader=None, trim_blocks=False, lstrip_blocks=False)
        self.env.globals.clear()
        self.env.globals["raise_exception"] = self._raise
        self.env.filters["tojson"] = lambda v, indent=None: json.dumps(v, ensure_ascii=False, indent=indent)
        try:
            self.template = self.env.from_string(source)
        except Exception as exc:
            raise ChatRenderError(f"template syntax error: {exc}") from None

    @staticmethod
    def _raise(msg):
        raise ChatRenderError(str(msg))

    def render(self, messages: list, add_generation_prompt: bool = True, **kwargs) -> str:
        ctx = {"messages": [{"role": m.role, "content": m.content, **({"reasoning_content": m.reasoning_content}
                                                                      if m.reasoning_content is not None else {})}
                            for m in messages],
               "add_generation_prompt": add_generation_prompt}
        ctx.update(json.loads(json.dumps(kwargs)))   # JSON-only context
        out, total, steps = [], 0, 0
        try:
            for piece in self.template.generate(**ctx):
                steps += 1
                total += len(piece.encode("utf-8"))
                if steps > TEMPLATE_FUEL or total > MAX_RENDER_BYTES:
                    raise ChatRenderError("template exceeded its render budget")
                out.append(piece)
        except ChatRenderError:
            raise
        except Exception as exc:
            raise ChatRenderError(f"template error: {type(exc).__name__}") from None
        return "".join(out)


FIM_TEMPLATE = "<|fim_prefix|>{prefix}<|fim_suffix|>{suffix}<|fim_middle|>"


def render_infill(prefix: str, suffix: str) -> str:
    return FIM_TEMPLATE.format(prefix=prefix, suffix=suffix)

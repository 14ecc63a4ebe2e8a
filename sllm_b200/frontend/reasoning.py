"""Reasoning support: the streaming <think> separator and the reasoning-budget controller.

Separator (docs/api/openai-compatibility.md "Thinking and separated reasoning"): recognises `<think>` and
`</think>` even when a tag crosses delta boundaries, never exposes the tags, and treats everything as reasoning
when generation ends before `</think>`.  Controller (crates/sllm-frontend/src/reasoning.rs:1-17): a budget of
1..4096 reasoning tokens after which the close marker is forced by intersecting the candidate mask with the
next token of the marker.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

OPEN, CLOSE = "<think>", "</think>"


class ReasoningSeparator:
    def __init__(self, starts_in_reasoning: bool = True):
        self.in_reasoning = starts_in_reasoning
        self.held = ""

    def push(self, delta: str):
        """Returns (reasoning_delta, content_delta)."""
        buf = self.held + delta
        self.held = ""
        r_out, c_out = [], []
        while buf:
            tag = CLOSE if self.in_reasoning else OPEN
            i = buf.find(tag)
            if i >= 0:
                (r_out if self.in_reasoning else c_out).append(buf[:i])
                buf = buf[i + len(tag):]
                self.in_reasoning = not self.in_reasoning
                if not self.in_reasoning:
                    buf = buf.lstrip("\n") if not c_out else buf
                continue
            keep = 0
            for k in range(min(len(tag) - 1, len(buf)), 0, -1):
                if buf.endswith(tag[:k]):
                    keep = k
                    break
            emit = buf[:len(buf) - keep] if keep else buf
            (r_out if self.in_reasoning else c_out).append(emit)
            self.held = buf[len(buf) - keep:] if keep else ""
            buf = ""
        return "".join(r_out), "".join(c_out)

    def flush(self):
        out, self.held = self.held, ""
        return (out, "") if self.in_reasoning else ("", out)


class ReasoningController:
    """Counts reasoning tokens; once the budget is spent it forces the close-marker token sequence."""

    def __init__(self, budget: int, close_marker_ids: Sequence[int], vocab: int, active: bool = True):
        if not 1 <= budget <= 4096:
            raise ValueError("reasoning budget must be in 1..4096")
        if not close_marker_ids:
            raise ValueError("close marker must tokenise to at least one token")
        self.budget, self.close, self.vocab = budget, list(close_marker_ids), vocab
        self.used = 0
        self.active = active
        self.forcing_at: Optional[int] = None
        self.matched = 0

    def mask(self) -> Optional[np.ndarray]:
        """Validity mask for the next token, or None when unconstrained."""
        if not self.active:
            return None
        if self.forcing_at is None and self.used >= self.budget:
            self.forcing_at = 0
        if self.forcing_at is None:
            return None
        m = np.zeros(self.vocab, dtype=np.uint8)
        m[self.close[self.forcing_at]] = 1
        return m

    def accept(self, token: int) -> None:
        if not self.active:
            return
        if self.forcing_at is not None:
            self.forcing_at += 1
            if self.forcing_at >= len(self.close):
                self.active = False
            return
        self.used += 1
        # the model may close the block by itself
        if token == self.close[self.matched]:
            self.matched += 1
            if self.matched == len(self.close):
                self.active = False
        else:
            self.matched = 1 if token == self.close[0] else 0

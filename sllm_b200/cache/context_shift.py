"""Context-window shift: a pure decision plus the engine-side rebuild.

Policy `disabled` fills the window exactly and fails closed on overflow.  Policy `keep_prefix_recent` compacts
whenever an append would fill or exceed the capacity: it keeps the first `keep_prefix` tokens and the last
`keep_recent` tokens, and the executor rebuilds a fresh KV state for the retained tokens (positions renumbered
from zero in the rebuilt state while the absolute position keeps counting).  The decision function touches no
backend state; the shift is a transaction that either commits the proposed state or leaves the old one
(reference: crates/sllm-core/src/context_window.rs:133-141 policy, :274-366 plan, :371-432 plan_initial).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

U64_MAX = (1 << 64) - 1


class ContextShiftError(ValueError):
    pass


@dataclass(frozen=True)
class WindowState:
    logical_length: int = 0        # tokens held by the KV state
    absolute_position: int = 0     # tokens ever appended
    shift_count: int = 0

    def validate(self):
        if self.logical_length > self.absolute_position:
            raise ContextShiftError("logical length exceeds the absolute position")

    def after_append(self, n: int, capacity: int) -> "WindowState":
        if self.logical_length + n > capacity:
            raise ContextShiftError("append exceeds the context capacity")
        if self.absolute_position + n > U64_MAX:
            raise ContextShiftError("position overflow")
        return WindowState(self.logical_length + n, self.absolute_position + n, self.shift_count)


@dataclass(frozen=True)
class ShiftDecision:
    shift: bool
    old_state: WindowState
    new_state: WindowState
    incoming: int
    prefix: tuple = (0, 0)         # [start, end) token ranges kept
    recent: tuple = (0, 0)

    def retained_token_ids(self, history: list) -> list:
        if not self.shift:
            return list(history)
        if len(history) != self.old_state.logical_length:
            raise ContextShiftError("token history does not match the window state")
        return list(history[self.prefix[0]:self.prefix[1]]) + list(history[self.recent[0]:self.recent[1]])

    def retained_absolute_positions(self) -> list:
        """Absolute positions of the retained tokens (prefix keeps its own; recent ends at the old end)."""
        base = self.old_state.absolute_position - self.old_state.logical_length
        return [base + i for i in range(*self.prefix)] + [base + i for i in range(*self.recent)]


@dataclass(frozen=True)
class ContextPolicy:
    kind: str = "disabled"         # disabled | keep_prefix_recent
    keep_prefix: int = 0
    keep_recent: int = 0
    version: int = 1

    @staticmethod
    def disabled() -> "ContextPolicy":
        return ContextPolicy()

    @staticmethod
    def keep_prefix_recent(keep_prefix: int, keep_recent: int) -> "ContextPolicy":
        if keep_prefix < 0 or keep_recent < 0 or keep_prefix + keep_recent == 0:
            raise ContextShiftError("the retained window must not be empty")
        return ContextPolicy("keep_prefix_recent", keep_prefix, keep_recent)

    @property
    def is_disabled(self) -> bool:
        return self.kind == "disabled"

    def identity(self) -> str:
        return "disabled" if self.is_disabled else f"kpr-v{self.version}:{self.keep_prefix}:{self.keep_recent}"

    def _validate(self):
        if self.version != 1 or self.kind not in ("disabled", "keep_prefix_recent"):
            raise ContextShiftError("unsupported context policy")

    def plan(self, state: WindowState, capacity: int, incoming: int) -> ShiftDecision:
        self._validate()
        state.validate()
        if capacity <= 0:
            raise ContextShiftError("capacity must be positive")
        if state.logical_length > capacity:
            raise ContextShiftError("state exceeds the capacity")
        required = state.logical_length + incoming
        if state.absolute_position + incoming > U64_MAX:
            raise ContextShiftError("position overflow")
        if incoming == 0 or required < capacity or (required == capacity and self.is_disabled):
            return ShiftDecision(False, state, state, incoming)
        if self.is_disabled:
            raise ContextShiftError("the context is full and shifting is disabled")
        L = state.logical_length
        if self.keep_prefix > L or self.keep_recent > L:
            raise ContextShiftError("a retained range exceeds the state")
        retained = self.keep_prefix + self.keep_recent
        if retained > L:
            raise ContextShiftError("retained ranges overlap")
        if retained + incoming > capacity:
            raise ContextShiftError("the retained window plus the incoming tokens exceed the capacity")
        new = WindowState(retained, state.absolute_position, state.shift_count + 1)
        return ShiftDecision(True, state, new, incoming, (0, self.keep_prefix), (L - self.keep_recent, L))

    def plan_initial(self, token_count: int, capacity: int) -> ShiftDecision:
        """Prompt-side counterpart: a prompt that already exceeds the capacity is compacted before prefill."""
        self._validate()
        if capacity <= 0:
            raise ContextShiftError("capacity must be positive")
        if token_count == 0:
            raise ContextShiftError("empty retained window")
        state = WindowState(token_count, token_count, 0)
        if token_count <= capacity:
            return ShiftDecision(False, state, state, 0)
        if self.is_disabled:
            raise ContextShiftError("the prompt exceeds the context and shifting is disabled")
        if self.keep_prefix > token_count or self.keep_recent > token_count:
            raise ContextShiftError("a retained range exceeds the prompt")
        retained = self.keep_prefix + self.keep_recent
        if retained == 0 or retained > capacity:
            raise ContextShiftError("the retained window exceeds the capacity")
        if retained > token_count:
            raise ContextShiftError("retained ranges overlap")
        return ShiftDecision(True, state, WindowState(retained, token_count, 1), 0, (0, self.keep_prefix),
                             (token_count - self.keep_recent, token_count))


def apply_shift(engine, seq, decision: ShiftDecision):
    """Rebuilds the KV state of `seq` for the retained tokens.  The prefix pages are shared with the old
    sequence by fork; the recent tokens are recomputed at their new positions.  The last retained token is left
    uncomputed so that the next decode step consumes it.  Returns the new sequence; the old one is freed only
    after the new state exists (transaction semantics)."""
    if not decision.shift:
        return seq
    kept = decision.retained_token_ids(seq.tokens[:decision.old_state.logical_length])
    tail = seq.tokens[decision.old_state.logical_length:]
    new = engine.fork_sequence(seq, kept) if decision.prefix[1] > 0 else engine.new_sequence(kept)
    try:
        new.prompt = list(kept)
        new.tokens = list(kept)
        if len(kept) - 1 > new.num_computed:
            # compute all retained tokens but the last; its KV is appended by the decode step that consumes it
            last = new.tokens.pop()
            engine.prefill([new], sample=False)
            new.tokens.append(last)
        new.tokens.extend(tail)
    except Exception:
        engine.free_sequence(new)
        raise
    new.user = seq.user
    engine.free_sequence(seq)
    return new

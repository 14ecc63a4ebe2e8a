"""Server lifecycle: loading -> ready -> draining -> shutdown, or failed (reference: lifecycle.rs)."""
from __future__ import annotations

import threading

STATES = ("loading", "ready", "draining", "failed", "shutdown")
_ALLOWED = {"loading": {"ready", "failed", "shutdown"}, "ready": {"draining", "failed", "shutdown"},
            "draining": {"shutdown", "failed"}, "failed": {"shutdown"}, "shutdown": set()}


class ServerLifecycle:
    def __init__(self):
        self._state = "loading"
        self._lock = threading.Lock()

    @property
    def state(self) -> str:
        return self._state

    def to(self, new: str) -> bool:
        with self._lock:
            if new in _ALLOWED[self._state]:
                self._state = new
                return True
            return False

    @property
    def ready(self) -> bool:
        return self._state == "ready"

"""Process-local replay buffer for resumable SSE: monotonic event ids, 64 KiB per event, 256 KiB per
session, bounded session and event counts, `Last-Event-ID` cursor (reference: crates/sllm-server/src/resume.rs:4-5)."""
from __future__ import annotations

import collections
import threading

MAX_EVENT_BYTES = 64 * 1024
MAX_SESSION_BYTES = 256 * 1024


class CursorTooOld(Exception):
    pass


class ReplaySession:
    def __init__(self, max_events: int):
        self.events = collections.deque()   # (id, bytes)
        self.bytes = 0
        self.next_id = 1
        self.first_id = 1
        self.closed = False
        self.max_events = max_events
        self.cond = threading.Condition()

    def append(self, data: bytes) -> int:
        if len(data) > MAX_EVENT_BYTES:
            raise ValueError("event exceeds 64 KiB")
        with self.cond:
            eid = self.next_id
            self.next_id += 1
            self.events.append((eid, data))
            self.bytes += len(data)
            while len(self.events) > self.max_events or self.bytes > MAX_SESSION_BYTES:
                _, old = self.events.popleft()
                self.bytes -= len(old)
                self.first_id = self.events[0][0] if self.events else self.next_id
            self.cond.notify_all()
            return eid

    def close(self):
        with self.cond:
            self.closed = True
            self.cond.notify_all()

    def after(self, cursor: int):
        with self.cond:
            if cursor + 1 < self.first_id:
                raise CursorTooOld()
            return [(i, d) for i, d in self.events if i > cursor], self.closed


class ResumableStore:
    def __init__(self, max_sessions: int = 64, max_events: int = 256):
        self.max_sessions, self.max_events = max_sessions, max_events
        self.sessions: "collections.OrderedDict[str, ReplaySession]" = collections.OrderedDict()
        self._lock = threading.Lock()

    def create(self, sid: str) -> ReplaySession:
        with self._lock:
            s = ReplaySession(self.max_events)
            self.sessions[sid] = s
            while len(self.sessions) > self.max_sessions:
                self.sessions.popitem(last=False)
            return s

    def get(self, sid: str):
        with self._lock:
            return self.sessions.get(sid)

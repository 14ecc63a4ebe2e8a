"""Model manifest and dynamic model lifecycle.

The manifest (`sllm-model-manifest-v1`) lists servable aliases with their GGUF path, derived lock and
per-model serving options.  The registry keeps at most `max_resident` models loaded, loads on first use
(concurrent requests for the same alias coalesce onto one load), hands out leases so a model in use is never
unloaded, evicts least-recently-used idle models, and quarantines an alias whose load failed until an operator
clears it.  States: unloaded -> loading -> ready -> draining -> unloaded, with failed / quarantined on errors
(reference: crates/sllm-server/src/model_lifecycle.rs, model_manifest.rs: <= 64 aliases, <= 16 resident).
"""
from __future__ import annotations

import json
import os
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Optional

from . import errors as E

MANIFEST_SCHEMA = "sllm-model-manifest-v1"
MAX_ALIASES = 64
MAX_RESIDENT = 16
MAX_MANIFEST_BYTES = 1024 * 1024
_ENTRY_KEYS = {"alias", "gguf", "derived_lock", "context_length", "kv_cache_encoding", "prefix_cache", "preload",
               "max_batch", "device_index", "tensor_parallel"}


class ManifestError(ValueError):
    pass


@dataclass
class ManifestEntry:
    alias: str
    gguf: str
    derived_lock: str
    context_length: Optional[int] = None
    kv_cache_encoding: Optional[str] = None
    prefix_cache: bool = False
    preload: bool = False
    max_batch: int = 64
    device_index: int = 0
    tensor_parallel: int = 1


def parse_manifest(data: bytes, base_dir: str = ".") -> list:
    if len(data) > MAX_MANIFEST_BYTES:
        raise ManifestError("manifest is too large")
    try:
        doc = json.loads(data.decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as exc:
        raise ManifestError(f"manifest is not valid JSON: {exc}") from None
    if not isinstance(doc, dict) or set(doc) != {"schema_version", "models"} or doc["schema_version"] != MANIFEST_SCHEMA:
        raise ManifestError("unknown manifest schema or unexpected top-level field")
    models = doc["models"]
    if not isinstance(models, list) or not 1 <= len(models) <= MAX_ALIASES:
        raise ManifestError("manifest must list 1..64 models")
    out, seen = [], set()
    for m in models:
        if not isinstance(m, dict) or set(m) - _ENTRY_KEYS:
            raise ManifestError("unknown field in a manifest entry")
        for k in ("alias", "gguf", "derived_lock"):
            if not isinstance(m.get(k), str) or not m[k]:
                raise ManifestError(f"manifest entry lacks {k}")
        alias = m["alias"]
        if alias in seen or len(alias) > 128 or any(c in alias for c in "/\\ \t\n"):
            raise ManifestError(f"invalid or duplicate alias {alias!r}")
        seen.add(alias)
        kv = m.get("kv_cache_encoding")
        if kv is not None and kv not in ("fp16", "bf16", "fp8", "fp8-static", "nvfp4"):
            raise ManifestError("unknown kv_cache_encoding")
        for k in ("context_length", "max_batch", "device_index", "tensor_parallel"):
            if k in m and (not isinstance(m[k], int) or isinstance(m[k], bool) or m[k] < 0):
                raise ManifestError(f"{k} must be a non-negative integer")
        res = lambda p: p if os.path.isabs(p) else os.path.join(base_dir, p)
        out.append(ManifestEntry(alias, res(m["gguf"]), res(m["derived_lock"]), m.get("context_length"), kv,
                                 bool(m.get("prefix_cache", False)), bool(m.get("preload", False)),
                                 m.get("max_batch", 64) or 64, m.get("device_index", 0), m.get("tensor_parallel", 1) or 1))
    return out


def read_manifest(path: str) -> list:
    with open(path, "rb") as f:
        return parse_manifest(f.read(MAX_MANIFEST_BYTES + 1), os.path.dirname(os.path.abspath(path)))


class Lease:
    def __init__(self, reg: "ModelLifecycleRegistry", slot: "_Slot"):
        self._reg, self._slot, self._done = reg, slot, False

    def release(self) -> None:
        if not self._done:
            self._done = True
            self._reg._release(self._slot)


@dataclass
class _Slot:
    entry: ManifestEntry
    state: str = "unloaded"     # unloaded | loading | ready | draining | failed | quarantined
    backend: object = None
    leases: int = 0
    last_used: float = 0.0
    error: str = ""
    loads: int = 0
    cond: threading.Condition = field(default_factory=threading.Condition)


class ModelLifecycleRegistry:
    """`loader(entry) -> backend` builds a backend (blocking); `unloader(backend)` tears it down."""

    def __init__(self, entries: list, loader: Callable, unloader: Optional[Callable] = None,
                 max_resident: int = MAX_RESIDENT, load_timeout_s: float = 600.0):
        if not 1 <= len(entries) <= MAX_ALIASES:
            raise ManifestError("1..64 aliases are supported")
        self.max_resident = max(1, min(max_resident, MAX_RESIDENT))
        self._slots = {e.alias: _Slot(e) for e in entries}
        self._loader, self._unloader = loader, unloader or (lambda b: getattr(b, "shutdown", lambda *a: None)())
        self._lock = threading.Lock()
        self.load_timeout_s = load_timeout_s

    # ------------------------------------------------------------------ queries
    def aliases(self) -> list:
        return list(self._slots)

    def states(self) -> dict:
        with self._lock:
            return {a: {"state": s.state, "leases": s.leases, "loads": s.loads, "error": s.error} for a, s in self._slots.items()}

    def resident(self) -> int:
        return sum(1 for s in self._slots.values() if s.state in ("ready", "loading", "draining"))

    # ------------------------------------------------------------------ acquire / release
    def acquire(self, alias: str):
        slot = self._slots.get(alias)
        if slot is None:
            raise E.model_not_found(alias)
        self._ensure_loaded(slot)
        with self._lock:
            if slot.state != "ready":
                raise E.ApiError(503, "model_unavailable", f"model {alias} is {slot.state}")
            slot.leases += 1
            slot.last_used = time.monotonic()
            return slot.backend, Lease(self, slot)

    def _release(self, slot: _Slot) -> None:
        with self._lock:
            slot.leases = max(0, slot.leases - 1)
            slot.last_used = time.monotonic()
        with slot.cond:
            slot.cond.notify_all()

    def _ensure_loaded(self, slot: _Slot) -> None:
        with self._lock:
            st = slot.state
            if st == "ready":
                return
            if st == "quarantined":
                raise E.ApiError(503, "model_quarantined", f"model {slot.entry.alias} is quarantined: {slot.error}")
            if st == "draining":
                raise E.ApiError(503, "model_unavailable", f"model {slot.entry.alias} is draining")
            leader = st in ("unloaded", "failed")
            if leader:
                if self.resident() >= self.max_resident and not self._evict_one_locked():
                    raise E.ApiError(503, "model_capacity", "all resident model slots are in use")
                slot.state = "loading"
        if leader:
            try:
                backend = self._loader(slot.entry)
            except Exception as exc:        # a failed load quarantines the alias until an operator clears it
                with self._lock:
                    slot.state, slot.error, slot.backend = "quarantined", f"{type(exc).__name__}: {exc}", None
                with slot.cond:
                    slot.cond.notify_all()
                raise E.ApiError(503, "model_load_failed", f"model {slot.entry.alias} failed to load") from None
            with self._lock:
                slot.backend, slot.state, slot.error = backend, "ready", ""
                slot.loads += 1
                slot.last_used = time.monotonic()
            with slot.cond:
                slot.cond.notify_all()
            return
        # follower: coalesce onto the load in progress
        end = time.monotonic() + self.load_timeout_s
        with slot.cond:
            while slot.state == "loading":
                left = end - time.monotonic()
                if left <= 0:
                    raise E.ApiError(503, "model_unavailable", "timed out waiting for the model to load")
                slot.cond.wait(min(left, 0.25))
        if slot.state != "ready":
            raise E.ApiError(503, "model_load_failed", f"model {slot.entry.alias} failed to load")

    # ------------------------------------------------------------------ eviction / admin
    def _evict_one_locked(self) -> bool:
        idle = [s for s in self._slots.values() if s.state == "ready" and s.leases == 0]
        if not idle:
            return False
        victim = min(idle, key=lambda s: s.last_used)
        self._unload_locked(victim)
        return True

    def _unload_locked(self, slot: _Slot) -> None:
        backend, slot.backend, slot.state = slot.backend, None, "unloaded"
        if backend is not None:
            try:
                self._unloader(backend)
            except Exception:
                pass

    def evict_idle(self) -> list:
        out = []
        with self._lock:
            for s in self._slots.values():
                if s.state == "ready" and s.leases == 0:
                    self._unload_locked(s)
                    out.append(s.entry.alias)
        return out

    def admin(self, alias: str, action: str) -> str:
        slot = self._slots[alias]
        if action in ("load", "preload"):
            self._ensure_loaded(slot)
        elif action == "unload":
            with self._lock:
                if slot.state == "ready":
                    slot.state = "draining"
            end = time.monotonic() + 30.0
            with slot.cond:
                while slot.leases > 0 and time.monotonic() < end:
                    slot.cond.wait(0.1)
            with self._lock:
                if slot.state == "draining":
                    if slot.leases > 0:
                        slot.state = "ready"
                        raise E.ApiError(409, "model_busy", f"model {alias} still has active requests")
                    self._unload_locked(slot)
        elif action == "clear-quarantine":
            with self._lock:
                if slot.state in ("quarantined", "failed"):
                    slot.state, slot.error = "unloaded", ""
        else:
            raise E.ApiError(404, "not_found", "unknown model action")
        return slot.state

    def preload_marked(self) -> None:
        for s in self._slots.values():
            if s.entry.preload:
                try:
                    self._ensure_loaded(s)
                except E.ApiError:
                    pass

    def shutdown(self) -> None:
        with self._lock:
            for s in self._slots.values():
                if s.backend is not None:
                    self._unload_locked(s)

"""Model lock: restricted-JSON parser, canonical fingerprint and hash-verified cache.

A model lock pins a source repository revision: every file with size and SHA-256, the architecture facts
the runtime depends on, the tokenizer contract and the generation stop policy.  The lock document is parsed
with a restricted JSON reader (size, depth, collection and string bounds; duplicate keys and floating-point
numbers rejected - numeric reals are carried as strings), its fingerprint is the SHA-256 of the RFC 8785
style canonical form of {schema_version, model} (object keys ordered by UTF-16 code units), and
`verify_cache` opens every listed file as a regular non-symlink file, checks size and digest through the
descriptor and keeps the descriptors open so later reads see the verified bytes
(reference: crates/sllm-core/src/model.rs:26-36 bounds, :599-720 verify_cache/parse, :2771-2830 fingerprint).
"""
from __future__ import annotations

import hashlib
import json
import os
import stat
from dataclasses import dataclass, field

MAX_LOCK_JSON_BYTES = 1024 * 1024
MAX_JSON_DEPTH = 64
MAX_JSON_ITEMS = 1_000_000
MAX_JSON_STRING_BYTES = 1024 * 1024
SAFE_INT = (1 << 53) - 1
SCHEMAS = ("model-lock-v1", "model-lock-v2")


class ModelLockError(ValueError):
    pass


def _pairs_no_dup(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise ModelLockError(f"duplicate object key {k!r}")
        out[k] = v
    return out


def _reject_float(text):
    raise ModelLockError("floating-point numbers are not allowed; carry reals as strings")


def _reject_const(text):
    raise ModelLockError("non-finite numbers are not allowed")


def _check(v, depth=0):
    if depth > MAX_JSON_DEPTH:
        raise ModelLockError("JSON nesting is too deep")
    if isinstance(v, str):
        if len(v.encode("utf-8")) > MAX_JSON_STRING_BYTES or any(ord(c) < 0x20 and c not in "\t\n\r" for c in v):
            raise ModelLockError("string is too long or contains control characters")
    elif isinstance(v, bool) or v is None:
        return
    elif isinstance(v, int):
        if abs(v) > SAFE_INT:
            raise ModelLockError("integer outside the safe range")
    elif isinstance(v, list):
        if len(v) > MAX_JSON_ITEMS:
            raise ModelLockError("array is too long")
        for x in v:
            _check(x, depth + 1)
    elif isinstance(v, dict):
        if len(v) > MAX_JSON_ITEMS:
            raise ModelLockError("object is too large")
        for k, x in v.items():
            _check(k, depth + 1)
            _check(x, depth + 1)


def parse_restricted_json(data: bytes, limit: int = MAX_LOCK_JSON_BYTES):
    if len(data) > limit:
        raise ModelLockError("document exceeds its size bound")
    try:
        text = data.decode("utf-8")
        v = json.loads(text, object_pairs_hook=_pairs_no_dup, parse_float=_reject_float, parse_constant=_reject_const)
    except (UnicodeDecodeError, json.JSONDecodeError, RecursionError) as exc:
        raise ModelLockError(f"invalid JSON: {exc}") from None
    _check(v)
    return v


def canonical_json(v) -> str:
    if v is None:
        return "null"
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, int):
        return str(v)
    if isinstance(v, str):
        return json.dumps(v, ensure_ascii=False)
    if isinstance(v, list):
        return "[" + ",".join(canonical_json(x) for x in v) + "]"
    if isinstance(v, dict):
        keys = sorted(v, key=lambda k: k.encode("utf-16-be"))
        return "{" + ",".join(json.dumps(k, ensure_ascii=False) + ":" + canonical_json(v[k]) for k in keys) + "}"
    raise ModelLockError("value cannot be canonicalised")


def fingerprint(doc: dict) -> str:
    body = {"schema_version": doc["schema_version"], "model": doc["model"]}
    return "sha256:" + hashlib.sha256(canonical_json(body).encode("utf-8")).hexdigest()


@dataclass
class LockedFile:
    path: str
    size_bytes: int
    sha256: str


@dataclass
class ModelLock:
    schema_version: str
    fingerprint: str
    aliases: list
    repo_id: str
    resolved_revision: str
    files: list
    architecture: dict
    tokenizer_contract: dict
    raw: dict = field(repr=False, default_factory=dict)

    @property
    def stop_token_ids(self) -> list:
        pol = self.tokenizer_contract.get("generation_stop_policy") or {}
        return list(pol.get("stop_token_ids", []))

    def verify_cache(self, root: str) -> "VerifiedCache":
        return VerifiedCache(self, root)


def parse_model_lock(data: bytes) -> ModelLock:
    doc = parse_restricted_json(data)
    if not isinstance(doc, dict) or doc.get("schema_version") not in SCHEMAS:
        raise ModelLockError("unknown model lock schema")
    for k in ("model", "fingerprint", "aliases"):
        if k not in doc:
            raise ModelLockError(f"model lock lacks {k}")
    m = doc["model"]
    if not isinstance(m, dict):
        raise ModelLockError("model section must be an object")
    if fingerprint(doc) != doc["fingerprint"]:
        raise ModelLockError("model lock fingerprint mismatch")
    files, seen = [], set()
    for f in m.get("files", []):
        p = f.get("path")
        if not isinstance(p, str) or not p or p.startswith("/") or ".." in p.split("/") or "\\" in p or p in seen:
            raise ModelLockError(f"unsafe or duplicate file path {p!r}")
        seen.add(p)
        sha = f.get("sha256")
        if not (isinstance(sha, str) and len(sha) == 64 and all(c in "0123456789abcdef" for c in sha)):
            raise ModelLockError("file digest must be lowercase hex SHA-256")
        if not isinstance(f.get("size_bytes"), int) or f["size_bytes"] < 0:
            raise ModelLockError("file size must be a non-negative integer")
        files.append(LockedFile(p, f["size_bytes"], sha))
    rev = m.get("resolved_revision", "")
    if not (isinstance(rev, str) and len(rev) == 40 and all(c in "0123456789abcdef" for c in rev)):
        raise ModelLockError("resolved revision must be a 40-hex commit id")
    aliases = doc["aliases"]
    if not (isinstance(aliases, list) and all(isinstance(a, str) and a for a in aliases)):
        raise ModelLockError("aliases must be non-empty strings")
    return ModelLock(doc["schema_version"], doc["fingerprint"], aliases, m.get("repo_id", ""), rev, files,
                     m.get("architecture", {}), m.get("tokenizer_contract", {}), doc)


def read_model_lock(path: str) -> ModelLock:
    st = os.lstat(path)
    if not stat.S_ISREG(st.st_mode) or st.st_size > MAX_LOCK_JSON_BYTES:
        raise ModelLockError("model lock must be a bounded regular file")
    with open(path, "rb") as f:
        return parse_model_lock(f.read(MAX_LOCK_JSON_BYTES + 1))


class VerifiedCache:
    """Open descriptors of every locked file, each checked for type, size and digest."""

    def __init__(self, lock: ModelLock, root: str):
        self.lock, self.root, self.fds = lock, root, {}
        try:
            for f in lock.files:
                full = os.path.join(root, f.path)
                st = os.lstat(full)
                if not stat.S_ISREG(st.st_mode):
                    raise ModelLockError(f"{f.path}: not a regular file")
                fd = os.open(full, os.O_RDONLY | getattr(os, "O_NOFOLLOW", 0))
                self.fds[f.path] = fd
                if os.fstat(fd).st_size != f.size_bytes:
                    raise ModelLockError(f"{f.path}: size differs from the lock")
                h, off = hashlib.sha256(), 0
                while off < f.size_bytes:
                    b = os.pread(fd, min(16 << 20, f.size_bytes - off), off)
                    if not b:
                        raise ModelLockError(f"{f.path}: short read")
                    h.update(b)
                    off += len(b)
                if h.hexdigest() != f.sha256:
                    raise ModelLockError(f"{f.path}: digest differs from the lock")
        except Exception:
            self.close()
            raise

    def read(self, path: str, limit: int = 64 << 20) -> bytes:
        fd = self.fds[path]
        size = os.fstat(fd).st_size
        if size > limit:
            raise ModelLockError(f"{path}: exceeds its read bound")
        return os.pread(fd, size, 0)

    def close(self):
        for fd in self.fds.values():
            try:
                os.close(fd)
            except OSError:
                pass
        self.fds = {}


def make_model_lock(root: str, repo_id: str, revision: str, aliases: list, architecture: dict,
                    tokenizer_contract: dict, schema: str = "model-lock-v2") -> dict:
    """Builds a lock document for a local directory (used by the converter and the tests)."""
    files = []
    for dirpath, _, names in sorted(os.walk(root)):
        for n in sorted(names):
            full = os.path.join(dirpath, n)
            rel = os.path.relpath(full, root).replace(os.sep, "/")
            with open(full, "rb") as f:
                data = f.read()
            files.append({"path": rel, "size_bytes": len(data), "sha256": hashlib.sha256(data).hexdigest()})
    doc = {"schema_version": schema, "aliases": list(aliases),
           "model": {"repo_id": repo_id, "resolved_revision": revision, "files": files,
                     "architecture": architecture, "tokenizer_contract": tokenizer_contract}}
    doc["fingerprint"] = fingerprint(doc)
    return doc

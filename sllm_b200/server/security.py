"""Bearer-key store: keys are kept only as SHA-256 digests, compared in constant time, with roles
user / admin, at most 32 keys, and atomic reload from a key file of `user:<token>` / `admin:<token>` lines
(reference: crates/sllm-server/src/security.rs:16-18,225-234,349-360)."""
from __future__ import annotations

import hashlib
import hmac
import os
import threading
from typing import Optional

MAX_KEYS = 32
MIN_TOKEN_BYTES, MAX_TOKEN_BYTES = 8, 512


class CredentialError(ValueError):
    pass


def _digest(token: str) -> bytes:
    return hashlib.sha256(token.encode("utf-8")).digest()


def parse_key_file(text: str) -> list:
    entries = []
    for raw in text.splitlines():
        line = raw.rstrip("\r")
        if not line or line.startswith("#"):
            continue
        if " " in line or "\t" in line or ":" not in line:
            raise CredentialError("key file lines must be role:token without spaces")
        role, token = line.split(":", 1)
        if role not in ("user", "admin"):
            raise CredentialError("unknown role in key file")
        if not MIN_TOKEN_BYTES <= len(token.encode()) <= MAX_TOKEN_BYTES:
            raise CredentialError("token length out of range")
        entries.append((role, _digest(token)))
    if not entries:
        raise CredentialError("key file holds no keys")
    if len(entries) > MAX_KEYS:
        raise CredentialError("too many keys")
    if len({d for _, d in entries}) != len(entries):
        raise CredentialError("duplicate key")
    return entries


class CredentialStore:
    """open() = no authentication for the user surface and NO admin access; from_user_key = one user-role key (the
    legacy ``--api-key-env`` configuration, which never administers models); from_key_file = explicit user / admin keys.
    Same separation as the reference (crates/sllm-server/src/security.rs:118-132 and its test at :406)."""

    def __init__(self, entries: Optional[list], path: Optional[str] = None):
        self._entries = entries
        self._path = path
        self._lock = threading.Lock()

    @classmethod
    def open(cls):
        return cls(None)

    @classmethod
    def from_user_key(cls, token: str):
        if not MIN_TOKEN_BYTES <= len(token.encode()) <= MAX_TOKEN_BYTES:
            raise CredentialError("token length out of range")
        return cls([("user", _digest(token))])

    @classmethod
    def from_key_file(cls, path: str):
        st = os.lstat(path)
        import stat
        if not stat.S_ISREG(st.st_mode):
            raise CredentialError("key file must be a regular, non-symlink file")
        with open(path, "r", encoding="utf-8") as f:
            return cls(parse_key_file(f.read()), path)

    @property
    def protected(self) -> bool:
        return self._entries is not None

    def role_for(self, authorization_header: Optional[str]) -> Optional[str]:
        """Returns 'admin', 'user' or None (rejected).  An open store makes every caller a user; admin always needs an
        explicit ``admin:`` key from a key file."""
        if self._entries is None:
            return "user"
        if not authorization_header or not authorization_header.startswith("Bearer "):
            return None
        d = _digest(authorization_header[7:])
        role = None
        with self._lock:
            for r, stored in self._entries:
                if hmac.compare_digest(d, stored):
                    role = r
        return role

    def reload(self) -> int:
        if self._path is None:
            raise CredentialError("the store was not loaded from a key file")
        fresh = CredentialStore.from_key_file(self._path)
        with self._lock:
            self._entries = fresh._entries
        return len(self._entries)

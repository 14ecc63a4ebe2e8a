"""`sllm models`: operator actions on a running server's dynamic model registry.

The server must be addressed over loopback cleartext (an API key never leaves the machine unencrypted);
actions: list, load, preload, unload, clear-quarantine, evict-idle (reference: crates/sllm-cli/src/model_admin.rs).
"""
from __future__ import annotations

import ipaddress
import json
import os
import urllib.error
import urllib.parse
import urllib.request

from .common import CliError, StrictParser, emit

ACTIONS = ("list", "load", "preload", "unload", "clear-quarantine", "evict-idle")


def _loopback(url: str) -> bool:
    u = urllib.parse.urlparse(url)
    if u.scheme != "http" or not u.hostname:
        return False
    if u.hostname == "localhost":
        return True
    try:
        return ipaddress.ip_address(u.hostname).is_loopback
    except ValueError:
        return False


def run_models(argv) -> int:
    p = StrictParser(prog="sllm models")
    p.add_argument("action", choices=ACTIONS)
    p.add_argument("alias", nargs="?")
    p.add_argument("--server", default="http://127.0.0.1:8080")
    p.add_argument("--api-key-env")
    p.add_argument("--api-key-file")
    a = p.parse_args(argv)
    if not _loopback(a.server):
        raise CliError("--server must be a loopback http:// address")
    if a.api_key_env and a.api_key_file:
        raise CliError("give at most one of --api-key-env and --api-key-file")
    key = None
    if a.api_key_env:
        key = os.environ.get(a.api_key_env)
        if not key:
            raise CliError(f"environment variable {a.api_key_env} is not set")
    elif a.api_key_file:
        with open(a.api_key_file, "r", encoding="utf-8") as f:
            key = f.read().strip()
    if a.action in ("load", "preload", "unload", "clear-quarantine") and not a.alias:
        raise CliError(f"{a.action} needs a model alias")
    base = a.server.rstrip("/")
    if a.action == "list":
        url, method = base + "/v1/models", "GET"
    elif a.action == "evict-idle":
        url, method = base + "/admin/models/evict-idle", "POST"
    else:
        url, method = f"{base}/admin/models/{urllib.parse.quote(a.alias, safe='')}/{a.action}", "POST"
    req = urllib.request.Request(url, method=method, data=b"" if method == "POST" else None)
    if key:
        req.add_header("Authorization", f"Bearer {key}")
    try:
        with urllib.request.urlopen(req, timeout=600) as r:
            emit(json.loads(r.read().decode("utf-8")))
            return 0
    except urllib.error.HTTPError as exc:
        try:
            emit(json.loads(exc.read().decode("utf-8")))
        except Exception:
            emit({"event": "error", "status": exc.code})
        return 1
    except (urllib.error.URLError, OSError) as exc:
        raise CliError(f"cannot reach the server: {exc}", 1) from None

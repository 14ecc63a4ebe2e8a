"""Session checkpoints: a little-endian, digest-protected envelope and a quota-bound store.

File layout (all integers little endian):
    0   8  magic "SB2CKPT1"
    8   2  schema version (1)         10  2  section count
    12  4  header bytes               16  8  total file bytes
    24  4  reserved (0)               28 32  SHA-256 of the whole file with this field zeroed
    60 36  reserved (0)               96 ..  identity block: 6 length-prefixed UTF-8 strings
                                             (model fingerprint, execution plan, KV layout, tokenizer,
                                              adapter, context policy), then the 32-byte token digest
    ..     section table: per section  u16 kind, u16 flags, u32 index, u64 offset, u64 length, 32-byte SHA-256
    ..     section payloads, each 32-byte aligned
Sections: 1 token history (u32 ids), 2 conversation (UTF-8 JSON), 3 state layers (JSON metadata), 4 state
planes (opaque native KV pages, one section per plane), 5 sampler state (JSON), 6 grammar state (JSON).
Decoding checks magic, version, bounds, table/payload overlap, every section digest, the file digest and
(optionally) that the identity matches the running model before any state is imported.  The store writes
to a temporary file in the same directory, fsyncs and renames (atomic replace), enforces a byte quota and
validates ids.  The envelope plays the role of the reference's `SLLMCKP1` container
(crates/sllm-core/src/session_checkpoint.rs:22-44 constants, :530-779 codec, :1332-1540 store) and protects the same
things, but it is NOT wire-compatible with it: the state planes are this engine's head-major KV pages, sections are
32-byte aligned and one per plane, and the identity block differs.  It therefore carries its own magic and schema id,
so that a file of either engine is rejected by the other as "not a session checkpoint" instead of as a malformed one.
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import struct
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

MAGIC = b"SB2CKPT1"
SCHEMA_VERSION = 1
SCHEMA_ID = "sllm-b200-session-checkpoint-v1"
MAX_HEADER_BYTES = 4096 + 56 * 4096
MAX_SECTIONS = 4096
MAX_CHECKPOINT_BYTES = 64 << 30
MAX_IDENTITY_FIELD_BYTES = 1024
MAX_TOKEN_HISTORY = 1 << 20
MAX_CONVERSATION_BYTES = 16 << 20
FIXED = 96
ENTRY = 56
S_TOKENS, S_CONVERSATION, S_LAYERS, S_PLANES, S_SAMPLER, S_GRAMMAR = 1, 2, 3, 4, 5, 6
_IDENTITY_FIELDS = ("model", "plan", "kv_layout", "tokenizer", "adapter", "context_policy")


class CheckpointError(ValueError):
    pass


def token_sequence_digest(tokens) -> bytes:
    return hashlib.sha256(np.asarray(tokens, dtype="<u4").tobytes()).digest()


@dataclass
class CheckpointIdentity:
    model: str = ""
    plan: str = ""
    kv_layout: str = ""
    tokenizer: str = ""
    adapter: str = ""
    context_policy: str = ""
    token_digest: bytes = b"\0" * 32

    def validate(self):
        for f in _IDENTITY_FIELDS:
            if len(getattr(self, f).encode("utf-8")) > MAX_IDENTITY_FIELD_BYTES:
                raise CheckpointError(f"identity field {f} is too long")
        if len(self.token_digest) != 32:
            raise CheckpointError("token digest must be 32 bytes")

    def encode(self) -> bytes:
        self.validate()
        out = bytearray()
        for f in _IDENTITY_FIELDS:
            b = getattr(self, f).encode("utf-8")
            out += struct.pack("<H", len(b)) + b
        return bytes(out + self.token_digest)


@dataclass
class SessionCheckpoint:
    identity: CheckpointIdentity
    tokens: list
    conversation: str = ""
    layers: dict = field(default_factory=dict)          # JSON-able metadata (shapes, dtype, length, page size)
    planes: list = field(default_factory=list)           # list[bytes]
    sampler_state: dict = field(default_factory=dict)
    grammar_state: dict = field(default_factory=dict)

    def encode(self) -> bytes:
        if len(self.tokens) > MAX_TOKEN_HISTORY:
            raise CheckpointError("token history is too long")
        conv = self.conversation.encode("utf-8")
        if len(conv) > MAX_CONVERSATION_BYTES:
            raise CheckpointError("conversation is too long")
        if token_sequence_digest(self.tokens) != self.identity.token_digest:
            raise CheckpointError("identity token digest does not match the token history")
        js = lambda o: json.dumps(o, sort_keys=True, separators=(",", ":")).encode("utf-8")
        secs = [(S_TOKENS, 0, np.asarray(self.tokens, dtype="<u4").tobytes()), (S_CONVERSATION, 0, conv),
                (S_LAYERS, 0, js(self.layers))]
        secs += [(S_PLANES, i, bytes(p)) for i, p in enumerate(self.planes)]
        secs += [(S_SAMPLER, 0, js(self.sampler_state)), (S_GRAMMAR, 0, js(self.grammar_state))]
        if len(secs) > MAX_SECTIONS:
            raise CheckpointError("too many sections")
        ident = self.identity.encode()
        header_bytes = FIXED + len(ident) + ENTRY * len(secs)
        off = (header_bytes + 31) // 32 * 32
        table = bytearray()
        body = bytearray()
        for kind, idx, payload in secs:
            table += struct.pack("<HHIQQ", kind, 0, idx, off, len(payload)) + hashlib.sha256(payload).digest()
            body += payload + b"\0" * ((-len(payload)) % 32)
            off += (len(payload) + 31) // 32 * 32
        total = off
        if total > MAX_CHECKPOINT_BYTES:
            raise CheckpointError("checkpoint is too large")
        head = bytearray(MAGIC + struct.pack("<HHIQI", SCHEMA_VERSION, len(secs), header_bytes, total, 0) + b"\0" * 68)
        out = head + ident + table
        out += b"\0" * ((-len(out)) % 32)
        out += body
        assert len(out) == total
        out[28:60] = hashlib.sha256(bytes(out)).digest()
        return bytes(out)

    @staticmethod
    def decode(data: bytes, expect: Optional[CheckpointIdentity] = None) -> "SessionCheckpoint":
        if len(data) < FIXED or data[:8] != MAGIC:
            raise CheckpointError("not a session checkpoint")
        ver, nsec, header_bytes, total, reserved = struct.unpack("<HHIQI", data[8:28])
        if ver != SCHEMA_VERSION:
            raise CheckpointError(f"unsupported checkpoint schema {ver}")
        if nsec > MAX_SECTIONS or header_bytes > MAX_HEADER_BYTES or header_bytes < FIXED or total != len(data) \
                or header_bytes > total or reserved != 0 or any(data[60:96]):
            raise CheckpointError("malformed checkpoint header")
        zeroed = bytearray(data)
        zeroed[28:60] = b"\0" * 32
        if hashlib.sha256(bytes(zeroed)).digest() != data[28:60]:
            raise CheckpointError("checkpoint digest mismatch")
        p = FIXED
        vals = {}
        for f in _IDENTITY_FIELDS:
            if p + 2 > header_bytes:
                raise CheckpointError("identity block is truncated")
            (n,) = struct.unpack("<H", data[p:p + 2])
            p += 2
            if n > MAX_IDENTITY_FIELD_BYTES or p + n > header_bytes:
                raise CheckpointError("identity field out of range")
            try:
                vals[f] = data[p:p + n].decode("utf-8")
            except UnicodeDecodeError:
                raise CheckpointError("identity field is not UTF-8") from None
            p += n
        if p + 32 + ENTRY * nsec != header_bytes:
            raise CheckpointError("header size does not match its contents")
        ident = CheckpointIdentity(token_digest=bytes(data[p:p + 32]), **vals)
        p += 32
        if expect is not None:
            for f in _IDENTITY_FIELDS:
                if getattr(expect, f) != getattr(ident, f):
                    raise CheckpointError(f"checkpoint identity mismatch: {f}")
        spans, parts = [], {}
        for _ in range(nsec):
            kind, flags, idx, off, ln = struct.unpack("<HHIQQ", data[p:p + 24])
            dig = data[p + 24:p + 56]
            p += ENTRY
            if flags != 0 or kind not in (1, 2, 3, 4, 5, 6) or off % 32 or off < header_bytes or off + ln > total:
                raise CheckpointError("section entry out of range")
            if (kind, idx) in parts or (kind != S_PLANES and idx != 0):
                raise CheckpointError("duplicate or misnumbered section")
            payload = bytes(data[off:off + ln])
            if hashlib.sha256(payload).digest() != dig:
                raise CheckpointError("section digest mismatch")
            spans.append((off, off + ln))
            parts[(kind, idx)] = payload
        spans.sort()
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            if b0 < a1:
                raise CheckpointError("sections overlap")
        for k in (S_TOKENS, S_CONVERSATION, S_LAYERS, S_SAMPLER, S_GRAMMAR):
            if (k, 0) not in parts:
                raise CheckpointError("a required section is missing")
        tk = parts[(S_TOKENS, 0)]
        if len(tk) % 4 or len(tk) // 4 > MAX_TOKEN_HISTORY:
            raise CheckpointError("token section malformed")
        tokens = np.frombuffer(tk, dtype="<u4").astype(np.int64).tolist()
        if token_sequence_digest(tokens) != ident.token_digest:
            raise CheckpointError("token digest mismatch")
        nplanes = sum(1 for k in parts if k[0] == S_PLANES)
        if sorted(i for k, i in parts if k == S_PLANES) != list(range(nplanes)):
            raise CheckpointError("plane sections are not contiguous")
        try:
            conv = parts[(S_CONVERSATION, 0)].decode("utf-8")
            layers = json.loads(parts[(S_LAYERS, 0)])
            sampler = json.loads(parts[(S_SAMPLER, 0)])
            grammar = json.loads(parts[(S_GRAMMAR, 0)])
        except (UnicodeDecodeError, json.JSONDecodeError):
            raise CheckpointError("a JSON section is malformed") from None
        return SessionCheckpoint(ident, tokens, conv, layers, [parts[(S_PLANES, i)] for i in range(nplanes)], sampler,
                                 grammar)


# ------------------------------------------------------------------------------------------ engine glue
def kv_layout_id(cache) -> str:
    s = cache.spec
    return f"paged{s.page_size}:{s.fmt}:L{s.n_layers}:H{s.kv_heads}:D{s.head_dim}"


def capture(engine, seq, identity: CheckpointIdentity, conversation: str = "", sampler_state: Optional[dict] = None,
            grammar_state: Optional[dict] = None) -> SessionCheckpoint:
    """Checkpoint of the computed part of `seq` (tokens beyond it are kept in the history and recomputed)."""
    import torch
    img = engine.cache.export_pages(seq.seq_id)
    vals = img["values"].contiguous()
    planes = [vals.reshape(-1).view(torch.uint8).numpy().tobytes()]
    layers = {"length": int(img["length"]), "values_shape": list(vals.shape), "values_dtype": str(vals.dtype),
              "kv_layout": kv_layout_id(engine.cache)}
    if "scales" in img:
        sc = img["scales"].contiguous()
        planes.append(sc.numpy().tobytes())
        layers["scales_shape"] = list(sc.shape)
    ident = CheckpointIdentity(identity.model, identity.plan, kv_layout_id(engine.cache), identity.tokenizer,
                               identity.adapter, identity.context_policy, token_sequence_digest(seq.tokens))
    return SessionCheckpoint(ident, list(seq.tokens), conversation, layers, planes, sampler_state or {},
                             grammar_state or {})


def restore(engine, ckpt: SessionCheckpoint):
    """Imports the KV pages into the pool and returns an engine sequence positioned after the computed tokens."""
    import torch
    from ..engine.engine import Sequence
    L = ckpt.layers
    if L.get("kv_layout") != kv_layout_id(engine.cache):
        raise CheckpointError("checkpoint KV layout does not match the running cache")
    dtype = {"torch.uint8": torch.uint8, "torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32,
             "torch.float16": torch.float16}[L["values_dtype"]]
    n = int(L["length"])
    if n > len(ckpt.tokens):
        raise CheckpointError("state length exceeds the token history")
    vals = torch.frombuffer(bytearray(ckpt.planes[0]), dtype=dtype).view(L["values_shape"])
    image = {"values": vals, "length": n}
    if "scales_shape" in L:
        image["scales"] = torch.frombuffer(bytearray(ckpt.planes[1]), dtype=torch.float32).view(L["scales_shape"])
    sid = engine.cache.import_pages(image)
    s = Sequence(prompt=list(ckpt.tokens))
    s.seq_id, s.num_computed = sid, n
    return s


# ------------------------------------------------------------------------------------------ store
_ID_RE = re.compile(r"^[A-Za-z0-9][A-Za-z0-9._-]{0,127}$")


class CheckpointStore:
    def __init__(self, root: str, max_bytes: int = 8 << 30, max_files: int = 1024):
        self.root, self.max_bytes, self.max_files = root, max_bytes, max_files
        os.makedirs(root, mode=0o700, exist_ok=True)
        if os.path.islink(root) or not os.path.isdir(root):
            raise CheckpointError("checkpoint root must be a real directory")

    def _path(self, cid: str) -> str:
        if not _ID_RE.match(cid) or ".." in cid:
            raise CheckpointError("invalid checkpoint id")
        return os.path.join(self.root, cid + ".ckpt")

    def usage_bytes(self) -> int:
        return sum(os.path.getsize(os.path.join(self.root, n)) for n in os.listdir(self.root) if n.endswith(".ckpt"))

    def list(self) -> list:
        return sorted(n[:-5] for n in os.listdir(self.root) if n.endswith(".ckpt"))

    def save(self, cid: str, ckpt: SessionCheckpoint) -> int:
        path = self._path(cid)
        data = ckpt.encode()
        old = os.path.getsize(path) if os.path.exists(path) else 0
        if self.usage_bytes() - old + len(data) > self.max_bytes:
            raise CheckpointError("checkpoint store quota exceeded")
        if not os.path.exists(path) and len(self.list()) >= self.max_files:
            raise CheckpointError("checkpoint store file limit reached")
        tmp = os.path.join(self.root, f".{cid}.{os.getpid()}.tmp")
        fd = os.open(tmp, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o600)
        try:
            with os.fdopen(fd, "wb") as f:
                f.write(data)
                f.flush()
                os.fsync(f.fileno())
            os.replace(tmp, path)
        except Exception:
            try:
                os.unlink(tmp)
            except OSError:
                pass
            raise
        return len(data)

    def load(self, cid: str, expect: Optional[CheckpointIdentity] = None) -> SessionCheckpoint:
        path = self._path(cid)
        st = os.lstat(path)
        import stat as _s
        if not _s.S_ISREG(st.st_mode) or st.st_size > MAX_CHECKPOINT_BYTES:
            raise CheckpointError("checkpoint must be a bounded regular file")
        with open(path, "rb") as f:
            return SessionCheckpoint.decode(f.read(), expect)

    def delete(self, cid: str) -> bool:
        try:
            os.unlink(self._path(cid))
            return True
        except FileNotFoundError:
            return False

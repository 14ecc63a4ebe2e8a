"""GGUF v3 container: bounded fail-closed reader, deterministic writer, sLLM tensor recipe, derived lock,
and the chunked verified weight upload.

Contract (reference: docs/formats/gguf.md, crates/sllm-core/src/gguf.rs:18-27,79-86,175-230,
gguf_writer.rs:529-536, weights.rs:21): magic `GGUF`, version 3, little endian, alignment 32, tensor rank
<= 4, tensor types F32(0) F16(1) I8 carrier(24) BF16(30) MXFP4(39, block 32 / 17 B) NVFP4(40, super-block
64 / 36 B); FP8 planes are I8 carriers bound to scale tensors through the versioned `sllm.tensor_recipe`
metadata (digest in `sllm.tensor_recipe.sha256`); tokenizer / chat template / frontend config live in the
same file.  The derived lock (`derived-gguf-lock-v1`) records output size and SHA-256, metadata and
tensor-catalog digests, the semantic model id and the source lock fingerprints.  The reader rejects
duplicate names, unknown types, overflow, overlap, ranges beyond EOF, bad alignment and rank > 4 before
any payload is touched; verification hashes the file through the descriptor that later serves the reads.
Weights are uploaded through one pinned 16 MiB staging chunk.
"""
from __future__ import annotations

import hashlib
import io
import json
import os
import struct
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

GGUF_MAGIC = b"GGUF"
GGUF_VERSION = 3
GGUF_ALIGNMENT = 32
MAX_HEADER_BYTES = 512 * 1024 * 1024
MAX_TENSORS = 1 << 20
MAX_KV = 1 << 16
UPLOAD_CHUNK_BYTES = 16 * 1024 * 1024

T_F32, T_F16, T_I8, T_BF16, T_MXFP4, T_NVFP4 = 0, 1, 24, 30, 39, 40
_BLOCK = {T_F32: (1, 4), T_F16: (1, 2), T_I8: (1, 1), T_BF16: (1, 2), T_MXFP4: (32, 17), T_NVFP4: (64, 36)}
(V_U8, V_I8, V_U16, V_I16, V_U32, V_I32, V_F32, V_BOOL, V_STR, V_ARR, V_U64, V_I64, V_F64) = range(13)
_SCALAR_FMT = {V_U8: "<B", V_I8: "<b", V_U16: "<H", V_I16: "<h", V_U32: "<I", V_I32: "<i", V_F32: "<f", V_BOOL: "<?",
               V_U64: "<Q", V_I64: "<q", V_F64: "<d"}

EXT_VERSION_KEY = "sllm.extension.version"
RECIPE_KEY = "sllm.tensor_recipe"
RECIPE_SHA_KEY = "sllm.tensor_recipe.sha256"
FRONTEND_CONFIG_KEY = "sllm.frontend.config_json"
FRONTEND_TOKENIZER_KEY = "sllm.frontend.tokenizer_json"
RECIPE_ENCODINGS = ("fp8-e4m3fn-channel-bf16-scale", "fp8-e4m3fn-channel-f32-scale", "fp8-e4m3fn-kblock128-f32-scale",
                    "nvfp4-e2m1-block16-e4m3fn-f32-outer", "mxfp4-e2m1-block32-e8m0")


class GgufError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    shape: tuple            # logical order (outermost first); GGUF stores dims innermost first
    ttype: int
    offset: int             # relative to the data section
    nbytes: int


def tensor_nbytes(shape: tuple, ttype: int) -> int:
    blk, bsz = _BLOCK[ttype]
    n = 1
    for d in shape:
        n *= d
    inner = shape[-1] if shape else 1
    if inner % blk:
        raise GgufError("innermost dimension is not a multiple of the block size")
    return n // blk * bsz


# ---------------------------------------------------------------------------------------------- block layouts
def mxfp4_to_gguf_blocks(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """[N, K/2] codes + [N, K/32] E8M0 -> [N, K/32, 17] (scale byte then 16 code bytes)."""
    n, kb = scales.shape
    out = np.empty((n, kb, 17), dtype=np.uint8)
    out[:, :, 0] = scales
    out[:, :, 1:] = packed.reshape(n, kb, 16)
    return out


def mxfp4_from_gguf_blocks(blocks: np.ndarray):
    n, kb, _ = blocks.shape
    return np.ascontiguousarray(blocks[:, :, 1:]).reshape(n, kb * 16), np.ascontiguousarray(blocks[:, :, 0])


def nvfp4_to_gguf_blocks(packed: np.ndarray, block_scales: np.ndarray) -> np.ndarray:
    """[N, K/2] codes + [N, K/16] E4M3 -> [N, K/64, 36] (four scale bytes then 32 code bytes)."""
    n, kb16 = block_scales.shape
    if kb16 % 4:
        raise GgufError("NVFP4 rows must be a multiple of 64 elements")
    sb = kb16 // 4
    out = np.empty((n, sb, 36), dtype=np.uint8)
    out[:, :, :4] = block_scales.reshape(n, sb, 4)
    out[:, :, 4:] = packed.reshape(n, sb, 32)
    return out


def nvfp4_from_gguf_blocks(blocks: np.ndarray):
    n, sb, _ = blocks.shape
    return np.ascontiguousarray(blocks[:, :, 4:]).reshape(n, sb * 32), np.ascontiguousarray(blocks[:, :, :4]).reshape(n, sb * 4)


# ---------------------------------------------------------------------------------------------- writer
def _w_str(buf: io.BytesIO, s: str):
    b = s.encode("utf-8")
    buf.write(struct.pack("<Q", len(b)))
    buf.write(b)


def _w_value(buf: io.BytesIO, v):
    if isinstance(v, bool):
        buf.write(struct.pack("<I", V_BOOL)); buf.write(struct.pack("<?", v))
    elif isinstance(v, int):
        if v < 0:
            buf.write(struct.pack("<I", V_I64)); buf.write(struct.pack("<q", v))
        elif v < (1 << 32):
            buf.write(struct.pack("<I", V_U32)); buf.write(struct.pack("<I", v))
        else:
            buf.write(struct.pack("<I", V_U64)); buf.write(struct.pack("<Q", v))
    elif isinstance(v, float):
        buf.write(struct.pack("<I", V_F32)); buf.write(struct.pack("<f", v))
    elif isinstance(v, str):
        buf.write(struct.pack("<I", V_STR)); _w_str(buf, v)
    elif isinstance(v, (list, tuple)):
        buf.write(struct.pack("<I", V_ARR))
        if all(isinstance(x, str) for x in v):
            buf.write(struct.pack("<IQ", V_STR, len(v)))
            for x in v:
                _w_str(buf, x)
        elif all(isinstance(x, int) and not isinstance(x, bool) for x in v):
            buf.write(struct.pack("<IQ", V_I32, len(v)))
            buf.write(np.asarray(v, dtype="<i4").tobytes())
        elif all(isinstance(x, float) for x in v):
            buf.write(struct.pack("<IQ", V_F32, len(v)))
            buf.write(np.asarray(v, dtype="<f4").tobytes())
        else:
            raise GgufError("arrays must be homogeneous strings, ints or floats")
    else:
        raise GgufError(f"unsupported metadata value type {type(v).__name__}")


def write_gguf(path: str, metadata: dict, tensors: list) -> dict:
    """tensors: list of (name, shape, ttype, bytes-like payload).  Deterministic: metadata keys are written in
    sorted order, tensors in the given order, padding is zero.  Returns digests for the derived lock."""
    names = [t[0] for t in tensors]
    if len(set(names)) != len(names):
        raise GgufError("duplicate tensor name")
    metadata = dict(metadata)
    metadata.setdefault("general.alignment", GGUF_ALIGNMENT)
    head = io.BytesIO()
    head.write(GGUF_MAGIC)
    head.write(struct.pack("<IQQ", GGUF_VERSION, len(tensors), len(metadata)))
    meta_buf = io.BytesIO()
    for k in sorted(metadata):
        _w_str(meta_buf, k)
        _w_value(meta_buf, metadata[k])
    head.write(meta_buf.getvalue())
    cat = io.BytesIO()
    off = 0
    for name, shape, ttype, payload in tensors:
        if len(shape) > 4 or ttype not in _BLOCK:
            raise GgufError("rank above 4 or unknown tensor type")
        nbytes = tensor_nbytes(tuple(shape), ttype)
        if len(payload) != nbytes:
            raise GgufError(f"payload size mismatch for {name}")
        _w_str(cat, name)
        cat.write(struct.pack("<I", len(shape)))
        for d in reversed(shape):
            cat.write(struct.pack("<Q", d))
        cat.write(struct.pack("<IQ", ttype, off))
        off = (off + nbytes + GGUF_ALIGNMENT - 1) // GGUF_ALIGNMENT * GGUF_ALIGNMENT
    head.write(cat.getvalue())
    header = head.getvalue()
    pad = (-len(header)) % GGUF_ALIGNMENT
    sha = hashlib.sha256()
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        for chunk in (header, b"\0" * pad):
            f.write(chunk); sha.update(chunk)
        for name, shape, ttype, payload in tensors:
            b = bytes(payload) if not isinstance(payload, (bytes, bytearray, memoryview)) else payload
            f.write(b); sha.update(b)
            p = (-len(b)) % GGUF_ALIGNMENT
            if p:
                f.write(b"\0" * p); sha.update(b"\0" * p)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)
    return {"size_bytes": os.path.getsize(path), "sha256": sha.hexdigest(),
            "metadata_sha256": hashlib.sha256(meta_buf.getvalue()).hexdigest(),
            "tensor_catalog_sha256": hashlib.sha256(cat.getvalue()).hexdigest()}


# ---------------------------------------------------------------------------------------------- reader
class _Cursor:
    def __init__(self, data: bytes):
        self.d, self.i = data, 0

    def take(self, n: int) -> bytes:
        if n < 0 or self.i + n > len(self.d):
            raise GgufError("truncated GGUF header")
        b = self.d[self.i:self.i + n]
        self.i += n
        return b

    def u32(self): return struct.unpack("<I", self.take(4))[0]
    def u64(self): return struct.unpack("<Q", self.take(8))[0]

    def string(self) -> str:
        n = self.u64()
        if n > MAX_HEADER_BYTES:
            raise GgufError("string length out of range")
        try:
            return self.take(n).decode("utf-8")
        except UnicodeDecodeError:
            raise GgufError("metadata string is not UTF-8") from None

    def value(self, vt: int, depth: int = 0):
        if vt in _SCALAR_FMT:
            fmt = _SCALAR_FMT[vt]
            return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]
        if vt == V_STR:
            return self.string()
        if vt == V_ARR:
            if depth:
                raise GgufError("nested arrays are not supported")
            et, n = self.u32(), self.u64()
            if n > MAX_HEADER_BYTES:
                raise GgufError("array length out of range")
            if et in _SCALAR_FMT and et != V_BOOL:
                fmt = _SCALAR_FMT[et]
                raw = self.take(n * struct.calcsize(fmt))
                return np.frombuffer(raw, dtype=np.dtype(fmt)).tolist()
            return [self.value(et, 1) for _ in range(n)]
        raise GgufError(f"unknown metadata value type {vt}")


class GgufFile:
    """An opened, structurally validated GGUF.  Payload reads go through the same descriptor."""

    def __init__(self, path: str):
        self.path = path
        st = os.lstat(path)
        import stat
        if not stat.S_ISREG(st.st_mode):
            raise GgufError("the model container must be a regular, non-symlink file")
        self.fd = os.open(path, os.O_RDONLY)
        try:
            self.size = os.fstat(self.fd).st_size
            self._parse()
        except Exception:
            os.close(self.fd)
            self.fd = -1
            raise

    def close(self):
        if self.fd >= 0:
            os.close(self.fd)
            self.fd = -1

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _parse(self):
        head = os.pread(self.fd, min(self.size, 24), 0)
        if len(head) < 24 or head[:4] != GGUF_MAGIC:
            raise GgufError("not a GGUF file")
        version, n_tensors, n_kv = struct.unpack("<IQQ", head[4:24])
        if version != GGUF_VERSION:
            raise GgufError(f"unsupported GGUF version {version}")
        if n_tensors > MAX_TENSORS or n_kv > MAX_KV:
            raise GgufError("tensor or metadata count out of range")
        # the header is read incrementally in bounded steps
        want = 1 << 20
        data = os.pread(self.fd, min(self.size, want), 0)
        while True:
            try:
                self._parse_header(data, n_tensors, n_kv)
                break
            except GgufError as exc:
                if "truncated" in str(exc) and len(data) < min(self.size, MAX_HEADER_BYTES):
                    want *= 4
                    data = os.pread(self.fd, min(self.size, want, MAX_HEADER_BYTES), 0)
                    continue
                raise

    def _parse_header(self, data: bytes, n_tensors: int, n_kv: int):
        c = _Cursor(data)
        c.take(24)
        meta_start = c.i
        md = {}
        for _ in range(n_kv):
            k = c.string()
            if k in md:
                raise GgufError(f"duplicate metadata key {k}")
            md[k] = c.value(c.u32())
        meta_end = c.i
        cat_start = c.i
        infos, seen = [], set()
        for _ in range(n_tensors):
            name = c.string()
            if name in seen:
                raise GgufError(f"duplicate tensor name {name}")
            seen.add(name)
            rank = c.u32()
            if rank > 4:
                raise GgufError("tensor rank above 4")
            dims = [c.u64() for _ in range(rank)]
            ttype, off = c.u32(), c.u64()
            if ttype not in _BLOCK:
                raise GgufError(f"unknown tensor type {ttype}")
            shape = tuple(reversed(dims))
            if any(d == 0 or d > (1 << 40) for d in shape):
                raise GgufError("tensor dimension out of range")
            infos.append(TensorInfo(name, shape, ttype, off, tensor_nbytes(shape, ttype)))
        cat_end = c.i
        align = md.get("general.alignment", GGUF_ALIGNMENT)
        if align != GGUF_ALIGNMENT:
            raise GgufError("alignment must be 32")
        self.data_start = (c.i + align - 1) // align * align
        spans = sorted((t.offset, t.offset + t.nbytes, t.name) for t in infos)
        prev_end = 0
        for b, e, name in spans:
            if b % align:
                raise GgufError(f"tensor {name} is not aligned")
            if b < prev_end:
                raise GgufError(f"tensor {name} overlaps another tensor")
            if self.data_start + e > self.size:
                raise GgufError(f"tensor {name} extends beyond the end of the file")
            prev_end = e
        self.metadata = md
        self.tensors = {t.name: t for t in infos}
        self.order = [t.name for t in infos]
        self.metadata_sha256 = hashlib.sha256(data[meta_start:meta_end]).hexdigest()
        self.tensor_catalog_sha256 = hashlib.sha256(data[cat_start:cat_end]).hexdigest()

    def sha256(self) -> str:
        h = hashlib.sha256()
        off = 0
        while off < self.size:
            b = os.pread(self.fd, min(UPLOAD_CHUNK_BYTES, self.size - off), off)
            if not b:
                raise GgufError("short read while hashing")
            h.update(b)
            off += len(b)
        return h.hexdigest()

    def read(self, name: str) -> bytes:
        t = self.tensors[name]
        b = os.pread(self.fd, t.nbytes, self.data_start + t.offset)
        if len(b) != t.nbytes:
            raise GgufError(f"short read for {name}")
        return b

    def numpy(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        raw = self.read(name)
        if t.ttype == T_F32:
            return np.frombuffer(raw, dtype="<f4").reshape(t.shape)
        if t.ttype == T_F16:
            return np.frombuffer(raw, dtype="<f2").reshape(t.shape)
        if t.ttype == T_BF16:
            return np.frombuffer(raw, dtype="<u2").reshape(t.shape)      # raw bf16 bits
        if t.ttype == T_I8:
            return np.frombuffer(raw, dtype=np.uint8).reshape(t.shape)
        blk, bsz = _BLOCK[t.ttype]
        return np.frombuffer(raw, dtype=np.uint8).reshape(t.shape[:-1] + (t.shape[-1] // blk, bsz))

    def upload(self, name: str, device, dtype=None):
        """Chunked upload through one pinned 16 MiB staging buffer; returns a flat uint8 device tensor
        (or a view of `dtype`)."""
        import torch
        t = self.tensors[name]
        out = torch.empty(t.nbytes, dtype=torch.uint8, device=device)
        pin = torch.device(device).type == "cuda"
        stage = torch.empty(min(UPLOAD_CHUNK_BYTES, max(t.nbytes, 1)), dtype=torch.uint8, pin_memory=pin)
        off = 0
        while off < t.nbytes:
            n = min(UPLOAD_CHUNK_BYTES, t.nbytes - off)
            b = os.pread(self.fd, n, self.data_start + t.offset + off)
            if len(b) != n:
                raise GgufError(f"short read for {name}")
            stage[:n].copy_(torch.frombuffer(bytearray(b), dtype=torch.uint8))
            out[off:off + n].copy_(stage[:n], non_blocking=False)
            off += n
        return out if dtype is None else out.view(dtype)

    def recipe(self) -> Optional[dict]:
        raw = self.metadata.get(RECIPE_KEY)
        if raw is None:
            return None
        if self.metadata.get(EXT_VERSION_KEY) != 1:
            raise GgufError("unknown sllm extension version")
        if hashlib.sha256(raw.encode("utf-8")).hexdigest() != self.metadata.get(RECIPE_SHA_KEY):
            raise GgufError("tensor recipe digest mismatch")
        rec = json.loads(raw)
        if rec.get("schema_version") != "sllm-tensor-recipe-v1":
            raise GgufError("unknown tensor recipe schema")
        used = set()
        for b in rec.get("bindings", []):
            if set(b) != {"logical_tensor", "value_tensor", "encoding", "role", "logical_shape", "scope", "scales"}:
                raise GgufError("malformed tensor binding")
            if b["encoding"] not in RECIPE_ENCODINGS or b["scope"] not in ("consumed", "known-unconsumed"):
                raise GgufError("unknown recipe encoding or scope")
            for n in [b["value_tensor"]] + [s["tensor"] for s in b["scales"]]:
                if n not in self.tensors:
                    raise GgufError(f"recipe names a missing tensor: {n}")
                if n in used:
                    raise GgufError(f"tensor bound twice: {n}")
                used.add(n)
        return rec


def recipe_metadata(bindings: list, static_fp8_kv: Optional[list] = None, known_unconsumed: Optional[list] = None) -> dict:
    rec = {"schema_version": "sllm-tensor-recipe-v1", "bindings": bindings, "logical_shapes": [],
           "static_fp8_kv": static_fp8_kv or []}
    if known_unconsumed:
        rec["known_unconsumed_tensors"] = sorted(known_unconsumed)
    raw = json.dumps(rec, sort_keys=True, separators=(",", ":"))
    return {EXT_VERSION_KEY: 1, RECIPE_KEY: raw, RECIPE_SHA_KEY: hashlib.sha256(raw.encode()).hexdigest()}


# ---------------------------------------------------------------------------------------------- derived lock
DERIVED_LOCK_SCHEMA = "derived-gguf-lock-v1"


def make_derived_lock(gguf_path: str, digests: dict, semantic_model_id: str, source_lock_fingerprints: list,
                      converter: dict) -> dict:
    body = {"schema_version": DERIVED_LOCK_SCHEMA, "semantic_model_id": semantic_model_id,
            "source_lock_fingerprints": list(source_lock_fingerprints), "converter": converter,
            "output": {"path": os.path.basename(gguf_path), **digests}}
    body["fingerprint"] = hashlib.sha256(json.dumps(body, sort_keys=True, separators=(",", ":")).encode()).hexdigest()
    return body


def read_derived_lock(path: str) -> dict:
    with open(path, "r", encoding="utf-8") as f:
        lock = json.load(f)
    need = {"schema_version", "fingerprint", "semantic_model_id", "source_lock_fingerprints", "converter", "output"}
    if not isinstance(lock, dict) or set(lock) != need or lock["schema_version"] != DERIVED_LOCK_SCHEMA:
        raise GgufError("malformed derived lock")
    if set(lock["output"]) != {"path", "size_bytes", "sha256", "metadata_sha256", "tensor_catalog_sha256"}:
        raise GgufError("malformed derived lock output section")
    body = {k: v for k, v in lock.items() if k != "fingerprint"}
    if hashlib.sha256(json.dumps(body, sort_keys=True, separators=(",", ":")).encode()).hexdigest() != lock["fingerprint"]:
        raise GgufError("derived lock fingerprint mismatch")
    return lock


def verify_gguf(path: str, lock: dict) -> GgufFile:
    """Opens, hashes and validates `path` against its derived lock; returns the verified open file."""
    g = GgufFile(path)
    out = lock["output"]
    if g.size != out["size_bytes"] or g.metadata_sha256 != out["metadata_sha256"] \
            or g.tensor_catalog_sha256 != out["tensor_catalog_sha256"] or g.sha256() != out["sha256"]:
        g.close()
        raise GgufError("the GGUF file does not match its derived lock")
    return g

"""LoRA adapters and control vectors: lock parsing, verified payloads, oracle and execution.

A LoRA lock names, per target projection, the rank and the byte offsets of A [rank, in] and B [out, rank]
(bf16, little endian) inside one payload file pinned by size and SHA-256; the delta is
y += scale * (alpha / rank) * B (A x).  A control-vector lock names a [layers, hidden] bf16 block that is added
to the residual stream of layers [layer_start, layer_end): h += scale * v[layer].  Both are bounded and fail
closed (unknown fields, non-finite scales, ranges outside the payload).  Execution on the GPU uses the dense
GEMM path for the two skinny products and the broadcast-add kernel
(reference: crates/sllm-core/src/adapter.rs:672-795 oracles and scale rule; execution
crates/sllm-core/src/qwen_execution.rs:5919-6200).
"""
from __future__ import annotations

import hashlib
import json
import math
import os
import stat
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..ops import reference as ref
from ..ops.core import LinearWeight

MAX_LOCK_BYTES = 1 << 20
MAX_PAYLOAD_BYTES = 4 << 30
MAX_RANK = 512
MAX_TARGETS = 4096
LORA_SCHEMA = "sllm-lora-lock-v1"
CV_SCHEMA = "sllm-control-vector-lock-v1"
TARGET_NAMES = ("qkv", "o", "gate_up", "down")


class AdapterError(ValueError):
    pass


def _checked_scale(scale: float) -> float:
    if not isinstance(scale, (int, float)) or not math.isfinite(scale) or abs(scale) > 64.0:
        raise AdapterError("adapter scale must be finite and within [-64, 64]")
    return float(scale)


def _read_payload(path: str, size: int, sha256: str) -> bytes:
    st = os.lstat(path)
    if not stat.S_ISREG(st.st_mode) or st.st_size != size or size > MAX_PAYLOAD_BYTES:
        raise AdapterError("adapter payload must be a regular file of the locked size")
    with open(path, "rb") as f:
        data = f.read()
    if hashlib.sha256(data).hexdigest() != sha256:
        raise AdapterError("adapter payload digest mismatch")
    return data


def _load_lock(path: str, schema: str, keys: set) -> dict:
    if os.path.getsize(path) > MAX_LOCK_BYTES:
        raise AdapterError("adapter lock is too large")
    with open(path, "r", encoding="utf-8") as f:
        d = json.load(f)
    if not isinstance(d, dict) or d.get("schema_version") != schema or set(d) != keys:
        raise AdapterError("unknown adapter lock schema or fields")
    return d


@dataclass
class LoraTarget:
    layer: int
    name: str
    rank: int
    in_features: int
    out_features: int
    a: torch.Tensor        # bf16 [rank, in]
    b: torch.Tensor        # bf16 [out, rank]


@dataclass
class LoraAdapter:
    alias: str
    alpha: float
    targets: dict = field(default_factory=dict)     # (layer, name) -> LoraTarget

    def effective_scale(self, rank: int, scale: float) -> float:
        s = _checked_scale(scale)
        if not math.isfinite(self.alpha) or self.alpha <= 0 or rank <= 0:
            raise AdapterError("LoRA alpha or rank is invalid")
        eff = s * (self.alpha / rank)
        if not math.isfinite(eff):
            raise AdapterError("LoRA effective scale is non-finite")
        return eff

    def to(self, device) -> "LoraAdapter":
        return LoraAdapter(self.alias, self.alpha, {k: LoraTarget(t.layer, t.name, t.rank, t.in_features, t.out_features,
                                                                  t.a.to(device), t.b.to(device)) for k, t in self.targets.items()})


def load_lora(lock_path: str, payload_path: Optional[str] = None) -> LoraAdapter:
    d = _load_lock(lock_path, LORA_SCHEMA, {"schema_version", "alias", "alpha", "payload", "targets"})
    pay = d["payload"]
    if set(pay) != {"path", "size_bytes", "sha256"}:
        raise AdapterError("malformed payload section")
    data = _read_payload(payload_path or os.path.join(os.path.dirname(lock_path), pay["path"]), pay["size_bytes"], pay["sha256"])
    if not isinstance(d["targets"], list) or not 1 <= len(d["targets"]) <= MAX_TARGETS:
        raise AdapterError("a LoRA lock lists 1..4096 targets")
    ad = LoraAdapter(str(d["alias"]), float(d["alpha"]))
    ad.effective_scale(1, 1.0)
    for t in d["targets"]:
        if set(t) != {"layer", "name", "rank", "in_features", "out_features", "a_offset", "b_offset"} or t["name"] not in TARGET_NAMES:
            raise AdapterError("malformed LoRA target")
        r, i, o = t["rank"], t["in_features"], t["out_features"]
        if not (1 <= r <= MAX_RANK and i > 0 and o > 0):
            raise AdapterError("LoRA rank or shape out of range")
        a0, b0 = t["a_offset"], t["b_offset"]
        if a0 < 0 or b0 < 0 or a0 + r * i * 2 > len(data) or b0 + o * r * 2 > len(data):
            raise AdapterError("LoRA tensor range is outside the payload")
        a = torch.from_numpy(np.frombuffer(data, dtype="<i2", count=r * i, offset=a0).copy()).view(torch.bfloat16).view(r, i)
        b = torch.from_numpy(np.frombuffer(data, dtype="<i2", count=o * r, offset=b0).copy()).view(torch.bfloat16).view(o, r)
        key = (int(t["layer"]), t["name"])
        if key in ad.targets:
            raise AdapterError("duplicate LoRA target")
        ad.targets[key] = LoraTarget(key[0], key[1], r, i, o, a, b)
    return ad


@dataclass
class ControlVector:
    alias: str
    layer_start: int
    layer_end: int
    vectors: torch.Tensor     # bf16 [layer_end - layer_start, hidden]

    def to(self, device) -> "ControlVector":
        return ControlVector(self.alias, self.layer_start, self.layer_end, self.vectors.to(device))


def load_control_vector(lock_path: str, payload_path: Optional[str] = None) -> ControlVector:
    d = _load_lock(lock_path, CV_SCHEMA, {"schema_version", "alias", "hidden_size", "layer_start", "layer_end", "vector_offset",
                                         "payload"})
    pay = d["payload"]
    data = _read_payload(payload_path or os.path.join(os.path.dirname(lock_path), pay["path"]), pay["size_bytes"], pay["sha256"])
    h, l0, l1, off = d["hidden_size"], d["layer_start"], d["layer_end"], d["vector_offset"]
    if not (h > 0 and 0 <= l0 < l1 and off >= 0) or off + (l1 - l0) * h * 2 > len(data):
        raise AdapterError("control-vector range is outside the payload")
    v = torch.from_numpy(np.frombuffer(data, dtype="<i2", count=(l1 - l0) * h, offset=off).copy()).view(torch.bfloat16)
    return ControlVector(str(d["alias"]), l0, l1, v.view(l1 - l0, h))


# ------------------------------------------------------------------------------------------ oracles (one row)
def apply_lora_oracle(t: LoraTarget, x_bf16: torch.Tensor, y_bf16: torch.Tensor, eff_scale: float) -> torch.Tensor:
    """y + eff_scale * B (A x) with fp32 accumulation in the reference's loop order, rounded to bf16 once."""
    proj = (t.a.float() * x_bf16.float().view(1, -1)).sum(dim=1)
    delta = (t.b.float() * proj.view(1, -1)).sum(dim=1)
    return (y_bf16.float() + eff_scale * delta).to(torch.bfloat16)


def apply_control_vector_oracle(cv: ControlVector, hidden_bf16: torch.Tensor, layer: int, scale: float) -> torch.Tensor:
    if not cv.layer_start <= layer < cv.layer_end or hidden_bf16.shape[-1] != cv.vectors.shape[1]:
        raise AdapterError("control-vector layer or hidden size is invalid")
    s = _checked_scale(scale)
    return (hidden_bf16.float() + s * cv.vectors[layer - cv.layer_start].float()).to(torch.bfloat16)


# ------------------------------------------------------------------------------------------ execution
class AdapterSet:
    """Adapters selected for a forward pass: [(LoraAdapter, scale)], [(ControlVector, scale)]."""

    def __init__(self, loras=(), control_vectors=()):
        self.loras = [(a, _checked_scale(s)) for a, s in loras]
        self.cvs = [(c, _checked_scale(s)) for c, s in control_vectors]
        if len(self.loras) > 4 or len(self.cvs) > 4:
            raise AdapterError("at most 4 LoRA adapters and 4 control vectors per request")

    def identity(self) -> str:
        return ";".join([f"lora:{a.alias}:{s}" for a, s in self.loras] + [f"cv:{c.alias}:{s}" for c, s in self.cvs])

    def lora_delta(self, layer: int, name: str, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        """y [T, out] += sum over adapters of scale * B (A x); x [T, in] bf16 (or fp32 on the CPU oracle path)."""
        for ad, scale in self.loras:
            t = ad.targets.get((layer, name))
            if t is None:
                continue
            if x.shape[1] != t.in_features or y.shape[1] != t.out_features:
                raise AdapterError("LoRA target shape does not match the projection")
            eff = ad.effective_scale(t.rank, scale)
            if x.is_cuda:
                p = ops.linear(x, LinearWeight("dense", t.a))                       # [T, rank]
                p = ops.elementwise("scalar_mul", p, s=eff)
                y = ops.linear(p, LinearWeight("dense", t.b), residual=y)          # y + p B^T
            else:
                p = x.float() @ t.a.float().t()
                y = (y.float() + eff * (p @ t.b.float().t())).to(y.dtype)
        return y

    def control(self, layer: int, h: torch.Tensor) -> torch.Tensor:
        for cv, scale in self.cvs:
            if cv.layer_start <= layer < cv.layer_end:
                v = cv.vectors[layer - cv.layer_start]
                if h.is_cuda:
                    sv = (v.float() * scale).to(torch.bfloat16)
                    h = ops.elementwise("broadcast_add", h, sv)
                else:
                    h = (h.float() + scale * v.float()).to(h.dtype)
        return h


def write_lora(dirpath: str, alias: str, alpha: float, targets: list) -> str:
    """targets: [(layer, name, A [rank, in], B [out, rank])]; writes payload + lock, returns the lock path."""
    blob, specs = bytearray(), []
    for layer, name, a, b in targets:
        a16, b16 = a.to(torch.bfloat16).contiguous(), b.to(torch.bfloat16).contiguous()
        a_off = len(blob)
        blob += a16.view(torch.int16).numpy().tobytes()
        b_off = len(blob)
        blob += b16.view(torch.int16).numpy().tobytes()
        specs.append({"layer": layer, "name": name, "rank": a16.shape[0], "in_features": a16.shape[1],
                      "out_features": b16.shape[0], "a_offset": a_off, "b_offset": b_off})
    os.makedirs(dirpath, exist_ok=True)
    with open(os.path.join(dirpath, alias + ".lora.bin"), "wb") as f:
        f.write(bytes(blob))
    lock = {"schema_version": LORA_SCHEMA, "alias": alias, "alpha": alpha, "targets": specs,
            "payload": {"path": alias + ".lora.bin", "size_bytes": len(blob), "sha256": hashlib.sha256(bytes(blob)).hexdigest()}}
    lp = os.path.join(dirpath, alias + ".lora.json")
    with open(lp, "w", encoding="utf-8") as f:
        json.dump(lock, f)
    return lp


def write_control_vector(dirpath: str, alias: str, layer_start: int, vectors: torch.Tensor) -> str:
    blob = vectors.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
    os.makedirs(dirpath, exist_ok=True)
    with open(os.path.join(dirpath, alias + ".cv.bin"), "wb") as f:
        f.write(blob)
    lock = {"schema_version": CV_SCHEMA, "alias": alias, "hidden_size": vectors.shape[1], "layer_start": layer_start,
            "layer_end": layer_start + vectors.shape[0], "vector_offset": 0,
            "payload": {"path": alias + ".cv.bin", "size_bytes": len(blob), "sha256": hashlib.sha256(blob).hexdigest()}}
    lp = os.path.join(dirpath, alias + ".cv.json")
    with open(lp, "w", encoding="utf-8") as f:
        json.dump(lock, f)
    return lp

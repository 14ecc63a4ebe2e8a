"""Container-neutral descriptors of a low-bit model and the importer of a mixed-precision checkpoint.

A quantised checkpoint is described by typed value / scale planes (which bytes hold the codes, which tensor holds
which scale and whether it is stored as a reciprocal), a per-layer static FP8 KV scale pair, and ONE recipe that says
which projection family uses which encoding:

    attention projections  FP8 E4M3FN weights with one BF16 scale per output channel, activations FP8 per token
    MLP projections        NVFP4 (E2M1 codes, E4M3 scale per 16 elements, FP32 outer scale), W4A4 in the source recipe
    KV cache               FP8 E4M3FN with one static scale per layer for K and one for V

The source container is a safetensors file written by a `compressed-tensors` exporter; execution consumes the planes,
so a GGUF file that carries the same planes produces the same descriptors.  The importer turns them into resident
weights: FP8 channel-scaled matrices become the 1x128 block-scaled form of the tcgen05 GEMM, NVFP4 matrices become
the tiled layout of the W4 GEMM (activations stay bf16 there: W4A16), static KV scales are bound per layer.

Reference: crates/sllm-core/src/quantized_model.rs:31-110 (descriptor types), :549-637 (recipe validation),
:685-863 (inventory), :887-910 (digest).  The reference pins one published checkpoint by hash; this importer checks
structure, shapes and the recipe of whatever checkpoint it is given.
"""
from __future__ import annotations

import enum
import hashlib
import json
import os
import struct
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

RECIPE_SCHEMA = "sllm-mixed-precision-recipe-v1"
MAX_HEADER_BYTES = 256 * 1024 * 1024
MAX_CONFIG_BYTES = 1024 * 1024


class QuantizedModelError(ValueError):
    pass


class TensorEncoding(enum.Enum):
    UNQUANTIZED_BF16 = "bf16"
    FP8_E4M3FN_CHANNEL_BF16_SCALE = "fp8-e4m3fn-channel-bf16-scale"
    NVFP4_E2M1_BLOCK16_E4M3FN_F32_OUTER = "nvfp4-e2m1-block16-e4m3fn-f32-outer"
    MXFP4_E2M1_BLOCK32_E8M0 = "mxfp4-e2m1-block32-e8m0"
    MXFP8_E4M3_BLOCK32_E8M0 = "mxfp8-e4m3-block32-e8m0"


class TensorRole(enum.Enum):
    EMBEDDING = "embedding"
    ATTENTION_PROJECTION = "attention-projection"
    MLP_PROJECTION = "mlp-projection"
    NORMALIZATION = "normalization"
    SCALAR = "scalar"
    KNOWN_UNCONSUMED = "known-unconsumed"


class ScalePlaneRole(enum.Enum):
    WEIGHT_BLOCK = "weight-block"
    WEIGHT_OUTER = "weight-outer"
    INPUT_OUTER = "input-outer"
    WEIGHT_CHANNEL = "weight-channel"


@dataclass(frozen=True)
class ScalePlane:
    role: ScalePlaneRole
    source_name: str
    dtype: str
    shape: tuple
    source_range: tuple          # [begin, end) inside the data section
    reciprocal: bool             # the stored number divides (compressed-tensors "global scale") instead of multiplying


@dataclass(frozen=True)
class TensorDescriptor:
    logical_name: str
    source_name: str
    role: TensorRole
    encoding: TensorEncoding
    logical_shape: tuple
    value_dtype: str
    value_shape: tuple
    value_range: tuple
    scale_planes: tuple = ()

    def plane(self, role: ScalePlaneRole) -> Optional[ScalePlane]:
        for p in self.scale_planes:
            if p.role == role:
                return p
        return None


@dataclass(frozen=True)
class StaticFp8KvScale:
    """Decode scales of one layer's K and V pages, kept as the BF16 bit patterns of the file."""
    key_bits: int
    value_bits: int

    @staticmethod
    def _f(bits: int) -> float:
        return struct.unpack("<f", struct.pack("<I", (bits & 0xFFFF) << 16))[0]

    @property
    def key(self) -> float:
        return self._f(self.key_bits)

    @property
    def value(self) -> float:
        return self._f(self.value_bits)


@dataclass(frozen=True)
class MixedPrecisionRecipe:
    attention_weight: TensorEncoding
    attention_input: str
    mlp_weight: TensorEncoding
    mlp_input: TensorEncoding
    kv_cache: str
    ignored: tuple
    schema_version: str = RECIPE_SCHEMA

    def to_dict(self) -> dict:
        return {"schema_version": self.schema_version, "attention_weight": self.attention_weight.value,
                "attention_input": self.attention_input, "mlp_weight": self.mlp_weight.value,
                "mlp_input": self.mlp_input.value, "kv_cache": self.kv_cache, "ignored": list(self.ignored)}


# ---------------------------------------------------------------------------------------------- recipe
def _check_spec(spec, bits: int, strategy: str, group: Optional[int], dynamic: Optional[bool], what: str) -> None:
    if not isinstance(spec, dict):
        raise QuantizedModelError(f"{what}: quantisation spec is absent")
    if spec.get("num_bits") != bits or spec.get("type") != "float" or spec.get("strategy") != strategy:
        raise QuantizedModelError(f"{what}: expected {bits}-bit float, strategy {strategy}")
    if group is not None and spec.get("group_size") != group:
        raise QuantizedModelError(f"{what}: expected group size {group}")
    if dynamic is not None and bool(spec.get("dynamic")) != dynamic and spec.get("dynamic") != ("local" if dynamic else False):
        raise QuantizedModelError(f"{what}: dynamic flag differs")
    if spec.get("symmetric") is False:
        raise QuantizedModelError(f"{what}: asymmetric quantisation is not supported")


def parse_recipe(config_json: bytes) -> MixedPrecisionRecipe:
    """Validates the `quantization_config` of a mixed-precision compressed-tensors checkpoint: group_0 = FP8 W8A8
    (channel weights, per-token dynamic inputs) on the attention projections, group_1 = NVFP4 (group 16) on the MLP
    projections, FP8 per-tensor static KV cache."""
    if len(config_json) > MAX_CONFIG_BYTES:
        raise QuantizedModelError("config JSON is too large")
    try:
        root = json.loads(config_json)
    except json.JSONDecodeError as exc:
        raise QuantizedModelError(f"config JSON: {exc}") from None
    q = root.get("quantization_config") if isinstance(root, dict) else None
    if not isinstance(q, dict):
        raise QuantizedModelError("quantization_config is absent")
    if (q.get("format"), q.get("quant_method"), q.get("quantization_status")) != ("mixed-precision", "compressed-tensors",
                                                                                   "compressed"):
        raise QuantizedModelError("mixed quantization identity differs")
    groups = q.get("config_groups")
    if not isinstance(groups, dict) or set(groups) != {"group_0", "group_1"}:
        raise QuantizedModelError("expected exactly the attention and the MLP quantisation group")
    g0, g1 = groups["group_0"], groups["group_1"]
    if g0.get("format") != "float-quantized" or g1.get("format") != "nvfp4-pack-quantized":
        raise QuantizedModelError("quantization group format differs")
    _check_spec(g0.get("weights"), 8, "channel", None, False, "attention weights")
    _check_spec(g0.get("input_activations"), 8, "token", None, True, "attention inputs")
    _check_spec(g1.get("weights"), 4, "tensor_group", 16, False, "MLP weights")
    _check_spec(g1.get("input_activations"), 4, "tensor_group", 16, None, "MLP inputs")
    _check_spec(q.get("kv_cache_scheme"), 8, "tensor", None, False, "KV cache")
    ignored = q.get("ignore")
    if not isinstance(ignored, list) or not all(isinstance(x, str) for x in ignored):
        raise QuantizedModelError("ignore selector is absent or not a list of names")
    return MixedPrecisionRecipe(TensorEncoding.FP8_E4M3FN_CHANNEL_BF16_SCALE, "dynamic-per-token-e4m3fn",
                                TensorEncoding.NVFP4_E2M1_BLOCK16_E4M3FN_F32_OUTER,
                                TensorEncoding.NVFP4_E2M1_BLOCK16_E4M3FN_F32_OUTER,
                                "static-per-layer-tensor-e4m3fn-bf16-decode-scale", tuple(ignored))


# ---------------------------------------------------------------------------------------------- safetensors
_ST_ITEM = {"U8": 1, "I8": 1, "F8_E4M3": 1, "BF16": 2, "F16": 2, "F32": 4, "I32": 4, "I64": 8, "F64": 8}


@dataclass(frozen=True)
class SafeTensorEntry:
    dtype: str
    shape: tuple
    begin: int
    end: int


def read_safetensors_header(path: str):
    """(entries by name, data_start) of a safetensors file, with every range checked: inside the file, sized
    dtype x shape, and no two tensors overlapping."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise QuantizedModelError("safetensors: truncated length prefix")
        n = struct.unpack("<Q", head)[0]
        if n > MAX_HEADER_BYTES or 8 + n > size:
            raise QuantizedModelError("safetensors: header length out of range")
        try:
            meta = json.loads(f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as exc:
            raise QuantizedModelError(f"safetensors: header JSON: {exc}") from None
    data_start, data_len = 8 + n, size - 8 - n
    out, spans = {}, []
    for name, e in meta.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape, (b, en) = e["dtype"], tuple(int(x) for x in e["shape"]), e["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise QuantizedModelError(f"safetensors: malformed entry {name!r}") from None
        if dtype not in _ST_ITEM or any(x < 0 for x in shape):
            raise QuantizedModelError(f"safetensors: {name}: unsupported dtype or negative extent")
        want = _ST_ITEM[dtype] * int(np.prod(shape, dtype=np.int64)) if shape else _ST_ITEM[dtype]
        if not (0 <= b <= en <= data_len) or en - b != want:
            raise QuantizedModelError(f"safetensors: {name}: byte range does not match dtype x shape")
        out[name] = SafeTensorEntry(dtype, shape, int(b), int(en))
        spans.append((int(b), int(en), name))
    spans.sort()
    for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
        if b1 < e0:
            raise QuantizedModelError(f"safetensors: {n0} and {n1} overlap")
    return out, data_start


def _require(header: dict, name: str, dtype: str, shape: tuple) -> SafeTensorEntry:
    e = header.get(name)
    if e is None:
        raise QuantizedModelError(f"{name}: tensor is absent")
    if e.dtype != dtype or tuple(e.shape) != tuple(shape):
        raise QuantizedModelError(f"{name}: expected {dtype}{list(shape)}, found {e.dtype}{list(e.shape)}")
    return e


# ---------------------------------------------------------------------------------------------- inventory
@dataclass
class ModelGeometry:
    n_layers: int
    d_model: int
    q_size: int
    kv_size: int
    ffn: int
    vocab: int
    prefix: str = "model.language_model"


@dataclass
class QuantizedModel:
    path: str
    data_start: int
    recipe: MixedPrecisionRecipe
    prefix: str = "model.language_model"
    tensors: dict = field(default_factory=dict)        # logical name -> TensorDescriptor
    kv_scales: dict = field(default_factory=dict)      # layer -> StaticFp8KvScale
    digest: str = ""

    def read_range(self, rng: tuple) -> bytes:
        b, e = rng
        if not 0 <= b <= e:
            raise QuantizedModelError("byte range is reversed")
        with open(self.path, "rb") as f:
            f.seek(self.data_start + b)
            raw = f.read(e - b)
        if len(raw) != e - b:
            raise QuantizedModelError("byte range reaches past the end of the file")
        return raw

    def read_scale(self, plane: ScalePlane) -> np.ndarray:
        """The multiplying form of a scale plane as fp32 (a reciprocal plane is inverted here, once)."""
        raw = self.read_range(plane.source_range)
        if plane.dtype == "F32":
            v = np.frombuffer(raw, dtype="<f4").astype(np.float32)
        elif plane.dtype == "BF16":
            v = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif plane.dtype == "F8_E4M3":
            return np.frombuffer(raw, dtype=np.uint8).reshape(plane.shape)       # codes: decoded by the consumer
        else:
            raise QuantizedModelError(f"{plane.source_name}: scale dtype {plane.dtype} is not supported")
        v = v.reshape(plane.shape)
        if plane.reciprocal:
            if not np.all(np.isfinite(v)) or np.any(v <= 0):
                raise QuantizedModelError(f"{plane.source_name}: reciprocal scale is not a positive finite number")
            v = (np.float32(1.0) / v).astype(np.float32)
        return v


def _attention_desc(header, base: str, rows: int, cols: int) -> TensorDescriptor:
    w = _require(header, base + ".weight", "F8_E4M3", (rows, cols))
    s = _require(header, base + ".weight_scale", "BF16", (rows, 1))
    return TensorDescriptor(base + ".weight", base + ".weight", TensorRole.ATTENTION_PROJECTION,
                            TensorEncoding.FP8_E4M3FN_CHANNEL_BF16_SCALE, (rows, cols), "F8_E4M3", (rows, cols),
                            (w.begin, w.end),
                            (ScalePlane(ScalePlaneRole.WEIGHT_CHANNEL, base + ".weight_scale", "BF16", (rows, 1),
                                        (s.begin, s.end), False),))


def _mlp_desc(header, base: str, rows: int, cols: int) -> TensorDescriptor:
    v = _require(header, base + ".weight_packed", "U8", (rows, cols // 2))
    b = _require(header, base + ".weight_scale", "F8_E4M3", (rows, (cols + 15) // 16))
    wo = _require(header, base + ".weight_global_scale", "F32", (1,))
    io = _require(header, base + ".input_global_scale", "F32", (1,))
    planes = (ScalePlane(ScalePlaneRole.WEIGHT_BLOCK, base + ".weight_scale", "F8_E4M3", (rows, (cols + 15) // 16), (b.begin, b.end), False),
              ScalePlane(ScalePlaneRole.WEIGHT_OUTER, base + ".weight_global_scale", "F32", (1,), (wo.begin, wo.end), True),
              ScalePlane(ScalePlaneRole.INPUT_OUTER, base + ".input_global_scale", "F32", (1,), (io.begin, io.end), True))
    return TensorDescriptor(base + ".weight", base + ".weight_packed", TensorRole.MLP_PROJECTION,
                            TensorEncoding.NVFP4_E2M1_BLOCK16_E4M3FN_F32_OUTER, (rows, cols), "U8", (rows, cols // 2),
                            (v.begin, v.end), planes)


def build_inventory(header: dict, geo: ModelGeometry, path: str, data_start: int):
    """Descriptors of every tensor the text decoder consumes, and the per-layer static KV scales.  Every tensor of
    the file must be consumed, be an `input_scale` of an FP8 projection (the inputs are quantised per token at run
    time) or lie outside the language model (towers this importer does not read): anything else is an error."""
    out, consumed, kv = {}, set(), {}
    p = geo.prefix

    def dense(name: str, shape: tuple, role: TensorRole):
        e = _require(header, name, "BF16", shape)
        out[name] = TensorDescriptor(name, name, role, TensorEncoding.UNQUANTIZED_BF16, shape, "BF16", shape, (e.begin, e.end))
        consumed.add(name)

    dense(f"{p}.embed_tokens.weight", (geo.vocab, geo.d_model), TensorRole.EMBEDDING)
    dense(f"{p}.norm.weight", (geo.d_model,), TensorRole.NORMALIZATION)
    for layer in range(geo.n_layers):
        lp = f"{p}.layers.{layer}"
        for proj, rows, cols in (("q", geo.q_size, geo.d_model), ("k", geo.kv_size, geo.d_model),
                                 ("v", geo.kv_size, geo.d_model), ("o", geo.d_model, geo.q_size)):
            base = f"{lp}.self_attn.{proj}_proj"
            d = _attention_desc(header, base, rows, cols)
            out[d.logical_name] = d
            consumed.update([base + ".weight", base + ".weight_scale"])
        for proj, rows, cols in (("gate", geo.ffn, geo.d_model), ("up", geo.ffn, geo.d_model), ("down", geo.d_model, geo.ffn)):
            base = f"{lp}.mlp.{proj}_proj"
            d = _mlp_desc(header, base, rows, cols)
            out[d.logical_name] = d
            consumed.update([base + s for s in (".weight_packed", ".weight_scale", ".weight_global_scale", ".input_global_scale")])
        for norm in ("input_layernorm", "post_attention_layernorm"):
            dense(f"{lp}.{norm}.weight", (geo.d_model,), TensorRole.NORMALIZATION)
        kn, vn = f"{lp}.self_attn.k_scale", f"{lp}.self_attn.v_scale"
        ke, ve = _require(header, kn, "BF16", (1,)), _require(header, vn, "BF16", (1,))
        consumed.update([kn, vn])
        with open(path, "rb") as f:
            bits = []
            for e in (ke, ve):
                f.seek(data_start + e.begin)
                bits.append(struct.unpack("<H", f.read(2))[0])
        sc = StaticFp8KvScale(bits[0], bits[1])
        if not (sc.key > 0 and sc.value > 0 and np.isfinite(sc.key) and np.isfinite(sc.value)):
            raise QuantizedModelError(f"layer {layer}: static KV scale is not a positive finite number")
        kv[layer] = sc
    for name in header:
        if name in consumed or name.endswith(".input_scale") or not name.startswith(p + "."):
            continue
        raise QuantizedModelError(f"{name}: tensor of the language model is not consumed by the recipe")
    return out, kv


def recipe_digest(recipe: MixedPrecisionRecipe, tensors: dict, kv: dict) -> str:
    """sha256 over the schema, every tensor's (name, encoding, logical shape) in name order and every layer's KV
    scale bits: two checkpoints with the same digest execute the same recipe on the same shapes."""
    h = hashlib.sha256()
    h.update(recipe.schema_version.encode())
    for name in sorted(tensors):
        t = tensors[name]
        h.update(t.logical_name.encode())
        h.update(t.encoding.value.encode())
        for extent in t.logical_shape:
            h.update(struct.pack("<Q", extent))
    for layer in sorted(kv):
        h.update(struct.pack("<IHH", layer, kv[layer].key_bits, kv[layer].value_bits))
    return "sha256:" + h.hexdigest()


def open_mixed_precision_checkpoint(root: str, geo: ModelGeometry) -> QuantizedModel:
    """Verifies `config.json` + `model.safetensors` under ``root`` and returns the descriptors."""
    cfg_path, st_path = os.path.join(root, "config.json"), os.path.join(root, "model.safetensors")
    if os.path.getsize(cfg_path) > MAX_CONFIG_BYTES:
        raise QuantizedModelError("config.json is too large")
    with open(cfg_path, "rb") as f:
        recipe = parse_recipe(f.read())
    header, data_start = read_safetensors_header(st_path)
    tensors, kv = build_inventory(header, geo, st_path, data_start)
    return QuantizedModel(st_path, data_start, recipe, geo.prefix, tensors, kv, recipe_digest(recipe, tensors, kv))


# ---------------------------------------------------------------------------------------------- resident weights
def load_resident(qm: QuantizedModel, cfg, device):
    """LlamaWeights of a verified mixed-precision checkpoint: attention projections as 1x128 block-scaled FP8
    (re-quantised from the channel-scaled codes), MLP projections as tiled NVFP4 for the W4A16 GEMM (codes and block
    scales bit-exact, outer scale inverted once), norms and embeddings as bf16.  Returns (weights, kv_scales) with
    kv_scales = [(k, v)] per layer for the `fp8-static` cache."""
    import torch
    from ..models.llama import LayerWeights, LlamaWeights
    from ..ops.core import LinearWeight
    from ..ops.w4 import W4Weight
    from . import codecs
    device = torch.device(device)
    p = qm.prefix

    def bf16(name):
        d = qm.tensors[name]
        raw = np.frombuffer(qm.read_range(d.value_range), dtype="<u2").reshape(d.value_shape)
        return torch.from_numpy(raw.astype(np.int16)).view(torch.bfloat16).to(device)

    def attn_rows(base):
        d = qm.tensors[base + ".weight"]
        codes = np.frombuffer(qm.read_range(d.value_range), dtype=np.uint8).reshape(d.value_shape)
        scale = qm.read_scale(d.plane(ScalePlaneRole.WEIGHT_CHANNEL)).reshape(-1)
        return codecs.dequantize_fp8_outer_rows(codes, scale)

    def fp8_linear(bases):
        w = np.concatenate([attn_rows(b) for b in bases], axis=0)
        return LinearWeight.from_dense(torch.from_numpy(w).to(torch.bfloat16), "fp8").to(device)

    def nvfp4_parts(base):
        d = qm.tensors[base + ".weight"]
        packed = np.frombuffer(qm.read_range(d.value_range), dtype=np.uint8).reshape(d.value_shape)
        block = qm.read_scale(d.plane(ScalePlaneRole.WEIGHT_BLOCK))
        outer = float(qm.read_scale(d.plane(ScalePlaneRole.WEIGHT_OUTER))[0])
        return packed, block, outer, d.logical_shape

    def nvfp4_linear(bases):
        parts = [nvfp4_parts(b) for b in bases]
        if len({round(x[2], 12) for x in parts}) == 1:
            packed = np.concatenate([x[0] for x in parts], axis=0)
            block = np.concatenate([x[1] for x in parts], axis=0)
            w4 = W4Weight.from_file_layout("nvfp4", packed, block, parts[0][3][1], [parts[0][2]], device)
        else:
            # fused rows carry one outer scale: matrices with different ones are re-quantised together
            dense = np.concatenate([codecs.dequantize_nvfp4(x[0], x[1], x[2], x[3][1]) for x in parts], axis=0)
            w4 = W4Weight.quantize("nvfp4", torch.from_numpy(dense), device, keep_file=False)
        return LinearWeight("w4", None, None, w4)

    layers = []
    for li in range(cfg.n_layers):
        lp = f"{p}.layers.{li}"
        a, m = f"{lp}.self_attn.", f"{lp}.mlp."
        layers.append(LayerWeights(
            attn_norm=bf16(f"{lp}.input_layernorm.weight"),
            qkv=fp8_linear([a + "q_proj", a + "k_proj", a + "v_proj"]),
            o=fp8_linear([a + "o_proj"]),
            mlp_norm=bf16(f"{lp}.post_attention_layernorm.weight"),
            gate_up=nvfp4_linear([m + "gate_proj", m + "up_proj"]),
            down=nvfp4_linear([m + "down_proj"])))
    embed = bf16(f"{p}.embed_tokens.weight")
    weights = LlamaWeights(embed, layers, bf16(f"{p}.norm.weight"), LinearWeight("dense", embed), 0)
    return weights, [(qm.kv_scales[li].key, qm.kv_scales[li].value) for li in range(cfg.n_layers)]

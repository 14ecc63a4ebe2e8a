"""GGUF <-> resident weights for the dense decoder family.

Export writes one GGUF with llama.cpp-style tensor names (`token_embd.weight`, `blk.N.attn_q.weight`, ...),
the model configuration, tokenizer and chat template in metadata, FP8 planes as I8 carriers bound to their
FP32 1x128 scale tensors through the tensor recipe, and returns the derived lock.  Load verifies the file
against the lock, uploads each tensor through the pinned staging chunk, shards it for this tensor-parallel
rank, concatenates q|k|v and gate|up, and transposes FP8 scales once into the layout the GEMM epilogue reads.
(Reference: QwenResidentModel::new_gguf, crates/sllm-core/src/qwen_execution.rs:960-1194, resident upload
crates/sllm-core/src/weights.rs:21; converter crates/sllm-core/src/gguf_convert.rs.)
"""
from __future__ import annotations

import json
from typing import Optional

import numpy as np
import torch

from ..formats import gguf as G
from ..ops.core import LinearWeight
from .config import ModelConfig
from .llama import LayerWeights, LlamaWeights

CONVERTER_ID = "sllm-b200-convert-gguf-v1"
FP8_ENCODING = "fp8-e4m3fn-kblock128-f32-scale"
FP8_CHANNEL_ENCODINGS = ("fp8-e4m3fn-channel-f32-scale", "fp8-e4m3fn-channel-bf16-scale")
NVFP4_ENCODING = "nvfp4-e2m1-block16-e4m3fn-f32-outer"
MXFP4_ENCODING = "mxfp4-e2m1-block32-e8m0"


# per-layer vectors only some families carry: (tensor name after `blk.N.`, LayerWeights field)
_OPTIONAL_LAYER_VECTORS = (("attn_q_norm.weight", "q_norm"), ("attn_k_norm.weight", "k_norm"),
                           ("post_attention_norm.weight", "post_attn_norm"), ("post_ffw_norm.weight", "post_mlp_norm"),
                           ("layer_output_scale.weight", "layer_scalar"))


def _bf16_bytes(t: torch.Tensor) -> bytes:
    return t.detach().to(torch.bfloat16).contiguous().cpu().view(torch.int16).numpy().tobytes()


def _f32_bytes(t: torch.Tensor) -> bytes:
    return t.detach().to(torch.float32).contiguous().cpu().numpy().tobytes()


def _u8_bytes(t: torch.Tensor) -> bytes:
    return t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes()


def export_llama_gguf(cfg: ModelConfig, w: LlamaWeights, path: str, tokenizer_json: Optional[str] = None,
                      chat_template: Optional[str] = None, source_fingerprints: tuple = (),
                      converter_args: Optional[dict] = None, mtp=None, vision=None, fp8_channel_scales: bool = False) -> dict:
    """Writes unsharded (tensor-parallel size 1) weights; returns the derived lock document.  ``mtp``
    (models.mtp.MtpWeights, dense) adds the multi-token-prediction component as `mtp.*` tensors.
    ``fp8_channel_scales`` writes FP8 projections with one FP32 scale per output row (the reference's "outer vector"
    form, re-quantised from the resident values) instead of 1x128 block scales."""
    tensors, bindings = [], []
    dense_t = G.T_F32 if cfg.weight_format == "fp32" else G.T_BF16
    dense_b = _f32_bytes if cfg.weight_format == "fp32" else _bf16_bytes

    def add_dense(name, t):
        tensors.append((name, tuple(t.shape), dense_t, dense_b(t)))

    def add_linear(name, lw: LinearWeight, r0: int, r1: int):
        if lw.kind == "fp8" and fp8_channel_scales:
            from ..formats import codecs
            codes, sc = codecs.quantize_fp8_outer_rows(lw.dequantized()[r0:r1].cpu().numpy())
            tensors.append((name, tuple(codes.shape), G.T_I8, np.ascontiguousarray(codes).tobytes()))
            tensors.append((name + ".scale", (codes.shape[0],), G.T_F32, np.asarray(sc, dtype="<f4").tobytes()))
            bindings.append({"logical_tensor": name, "value_tensor": name, "encoding": FP8_CHANNEL_ENCODINGS[0],
                             "role": "weight", "logical_shape": list(codes.shape), "scope": "consumed",
                             "scales": [{"role": "channel", "tensor": name + ".scale"}]})
        elif lw.kind == "fp8":
            val = lw.w[r0:r1]
            sc = lw.scale_t[:, r0:r1].t().contiguous()          # file layout [N, ceil(K/128)]
            tensors.append((name, tuple(val.shape), G.T_I8, _u8_bytes(val)))
            tensors.append((name + ".scale", tuple(sc.shape), G.T_F32, _f32_bytes(sc)))
            bindings.append({"logical_tensor": name, "value_tensor": name, "encoding": FP8_ENCODING, "role": "weight",
                             "logical_shape": list(val.shape), "scope": "consumed",
                             "scales": [{"role": "block", "tensor": name + ".scale"}]})
        elif lw.kind == "w4":
            # 4-bit weights travel as standard GGML blocks (MXFP4 type 39, NVFP4 type 40); an NVFP4 tensor also binds
            # its FP32 tensor ("outer") scale (reference: gguf_convert.rs:33-96, recipe encodings gguf.rs:175-180)
            from ..formats import codecs
            w4 = lw.w4
            packed, scales = w4.to_file_layout(0)
            packed, scales = packed[r0:r1], scales[r0:r1]
            shape = (r1 - r0, w4.k)
            if w4.fmt == "mxfp4":
                tensors.append((name, shape, G.T_MXFP4, codecs.to_ggml_mxfp4(packed, scales, w4.k)))
                bindings.append({"logical_tensor": name, "value_tensor": name, "encoding": MXFP4_ENCODING, "role": "weight",
                                 "logical_shape": list(shape), "scope": "consumed", "scales": []})
            else:
                tensors.append((name, shape, G.T_NVFP4, codecs.to_ggml_nvfp4(packed, scales, w4.k)))
                tensors.append((name + ".outer_scale", (1,), G.T_F32, _f32_bytes(w4.tensor_scale[:1])))
                bindings.append({"logical_tensor": name, "value_tensor": name, "encoding": NVFP4_ENCODING, "role": "weight",
                                 "logical_shape": list(shape), "scope": "consumed",
                                 "scales": [{"role": "outer", "tensor": name + ".outer_scale"}]})
        else:
            add_dense(name, lw.w[r0:r1])

    add_dense("token_embd.weight", w.embed)
    q, kv, f = cfg.q_size, cfg.kv_size, cfg.ffn
    for i, l in enumerate(w.layers):
        p = f"blk.{i}."
        add_dense(p + "attn_norm.weight", l.attn_norm)
        add_linear(p + "attn_q.weight", l.qkv, 0, q)
        add_linear(p + "attn_k.weight", l.qkv, q, q + kv)
        add_linear(p + "attn_v.weight", l.qkv, q + kv, q + 2 * kv)
        add_linear(p + "attn_output.weight", l.o, 0, cfg.d_model)
        add_dense(p + "ffn_norm.weight", l.mlp_norm)
        add_linear(p + "ffn_gate.weight", l.gate_up, 0, f)
        add_linear(p + "ffn_up.weight", l.gate_up, f, 2 * f)
        add_linear(p + "ffn_down.weight", l.down, 0, cfg.d_model)
        for name, t in _OPTIONAL_LAYER_VECTORS:
            if getattr(l, t) is not None:
                add_dense(p + name, getattr(l, t))
    add_dense("output_norm.weight", w.final_norm)
    if not cfg.tie_embeddings:
        add_linear("output.weight", w.lm_head, 0, cfg.vocab)
    if vision is not None:              # models.vision_tower.VisionWeights: the 297-tensor inventory as `v.*`
        for name, t in vision_tensor_list(vision):
            add_dense(name, t)
    if mtp is not None:
        l = mtp.layer
        add_dense("mtp.fc.weight", mtp.fc.w)
        add_dense("mtp.pre_fc_norm_embedding.weight", mtp.norm_embedding)
        add_dense("mtp.pre_fc_norm_hidden.weight", mtp.norm_hidden)
        add_dense("mtp.norm.weight", mtp.norm)
        for name, t in (("attn_norm", l.attn_norm), ("attn_qkv", l.qkv.w), ("attn_output", l.o.w),
                        ("ffn_norm", l.mlp_norm), ("ffn_gate_up", l.gate_up.w), ("ffn_down", l.down.w)):
            add_dense(f"mtp.blk.0.{name}.weight", t)
    md = {"general.architecture": "llama", "general.name": cfg.name,
          "llama.block_count": cfg.n_layers, "llama.embedding_length": cfg.d_model,
          "llama.attention.head_count": cfg.n_heads, "llama.attention.head_count_kv": cfg.n_kv_heads,
          "llama.feed_forward_length": cfg.ffn, "llama.context_length": cfg.max_context,
          "llama.rope.freq_base": float(cfg.rope_theta), "llama.attention.layer_norm_rms_epsilon": float(cfg.rms_eps),
          G.FRONTEND_CONFIG_KEY: json.dumps(cfg.to_dict(), sort_keys=True)}
    if tokenizer_json is not None:
        md[G.FRONTEND_TOKENIZER_KEY] = tokenizer_json
    if chat_template is not None:
        md["tokenizer.chat_template"] = chat_template
    md.update(G.recipe_metadata(bindings))
    digests = G.write_gguf(path, md, tensors)
    return G.make_derived_lock(path, digests, f"{cfg.name}:{cfg.weight_format}", list(source_fingerprints),
                               {"id": CONVERTER_ID, "args": converter_args or {}})


def config_from_gguf(g: G.GgufFile) -> ModelConfig:
    raw = g.metadata.get(G.FRONTEND_CONFIG_KEY)
    if raw is None:
        raise G.GgufError("the GGUF file carries no model configuration")
    d = json.loads(raw)
    known = set(ModelConfig.__dataclass_fields__)
    if set(d) - known:
        raise G.GgufError(f"unknown configuration fields: {sorted(set(d) - known)}")
    return ModelConfig(**d)


def load_llama_gguf(g: G.GgufFile, device, tp_size: int = 1, tp_rank: int = 0, kv_format: Optional[str] = None):
    """Returns (cfg, LlamaWeights) for this rank from a verified open GGUF file."""
    cfg = config_from_gguf(g)
    if kv_format:
        cfg.kv_format = kv_format
    rec = g.recipe() or {"bindings": []}
    bound = {b["logical_tensor"]: b for b in rec["bindings"]}
    device = torch.device(device)
    hd = cfg.head_dim
    dense_dtype = torch.float32 if cfg.weight_format == "fp32" else torch.bfloat16

    def dense(name):
        t = g.tensors[name]
        want = G.T_F32 if dense_dtype == torch.float32 else G.T_BF16
        if t.ttype != want:
            raise G.GgufError(f"{name}: unexpected tensor type {t.ttype}")
        return g.upload(name, device, dense_dtype).view(t.shape)

    def rows(name, lo: int, hi: int, cols=None):
        """(values[lo:hi, cols], scales[lo:hi, cols/128] or None)."""
        t = g.tensors[name]
        b = bound.get(name)
        if b is None:
            v = dense(name)
            v = v[lo:hi] if cols is None else v[lo:hi, cols[0]:cols[1]]
            return v, None
        enc = b["encoding"]
        if enc in (NVFP4_ENCODING, MXFP4_ENCODING):
            return w4_rows(name, t, b, lo, hi, cols)
        if enc in FP8_CHANNEL_ENCODINGS and t.ttype == G.T_I8:
            # one scale per output row ("outer vector", the form the reference executes: fp8.rs:201): the same scale
            # for every 128-wide K block is the block-scaled form of it, exactly
            v = g.upload(name, device, torch.uint8).view(t.shape)
            sname = b["scales"][0]["tensor"]
            st = g.tensors[sname]
            if st.ttype == G.T_BF16:
                sv = g.upload(sname, device, torch.bfloat16).float()
            elif st.ttype == G.T_F32:
                sv = g.upload(sname, device, torch.float32)
            else:
                raise G.GgufError(f"{sname}: unexpected scale tensor type {st.ttype}")
            if sv.numel() != t.shape[0]:
                raise G.GgufError(f"{sname}: expected one scale per output row")
            s = sv.view(-1, 1).expand(t.shape[0], (t.shape[1] + 127) // 128).contiguous()
        elif enc == FP8_ENCODING and t.ttype == G.T_I8:
            v = g.upload(name, device, torch.uint8).view(t.shape)
            sname = b["scales"][0]["tensor"]
            s = g.upload(sname, device, torch.float32).view(g.tensors[sname].shape)
        else:
            raise G.GgufError(f"{name}: unsupported encoding {enc}")
        if cols is None:
            return v[lo:hi], s[lo:hi]
        if cols[0] % 128 or cols[1] % 128:
            raise G.GgufError("tensor-parallel column shards of FP8 weights must align to 128")
        return v[lo:hi, cols[0]:cols[1]], s[lo:hi, cols[0] // 128:cols[1] // 128]

    def w4_rows(name, t, b, lo, hi, cols):
        """A row / column range of a 4-bit tensor as ("w4", fmt, packed, scales, tensor_scale, k)."""
        from ..formats import codecs
        n, k = t.shape
        raw = g.upload(name, "cpu", torch.uint8).numpy().tobytes()
        if b["encoding"] == MXFP4_ENCODING:
            if t.ttype != G.T_MXFP4:
                raise G.GgufError(f"{name}: MXFP4 binding on tensor type {t.ttype}")
            fmt, blk, ts = "mxfp4", 32, None
            packed, scales = codecs.from_ggml_mxfp4(raw, n, k)
        else:
            if t.ttype != G.T_NVFP4:
                raise G.GgufError(f"{name}: NVFP4 binding on tensor type {t.ttype}")
            outer = [x for x in b.get("scales", []) if x.get("role") == "outer"]
            if len(outer) != 1:
                raise G.GgufError(f"{name}: an NVFP4 binding needs exactly one outer scale")
            fmt, blk = "nvfp4", 16
            ts = float(g.upload(outer[0]["tensor"], "cpu", torch.float32)[0])
            packed, scales = codecs.from_ggml_nvfp4(raw, n, k)
        packed, scales = packed[lo:hi], scales[lo:hi]
        if cols is not None:
            if cols[0] % 128 or cols[1] % 128:
                raise G.GgufError("tensor-parallel column shards of 4-bit weights must align to 128")
            packed, scales, k = packed[:, cols[0] // 2:cols[1] // 2], scales[:, cols[0] // blk:cols[1] // blk], cols[1] - cols[0]
        return ("w4", fmt, np.ascontiguousarray(packed), np.ascontiguousarray(scales), ts, k)

    def lin_w4(parts) -> LinearWeight:
        from ..formats import codecs
        from ..ops.w4 import W4Weight
        fmt, k = parts[0][1], parts[0][5]
        scales_equal = all(p[4] == parts[0][4] for p in parts)
        if scales_equal:          # one tensor scale (or none): the file bytes are used as they are
            packed = np.concatenate([p[2] for p in parts], axis=0)
            sc = np.concatenate([p[3] for p in parts], axis=0)
            return LinearWeight("w4", None, None, W4Weight.from_file_layout(fmt, packed, sc, k, parts[0][4], device))
        # q | k | v (or gate | up) quantised with different NVFP4 tensor scales share one matrix here: the values are
        # exact in fp32, so the fused matrix is re-quantised once with a common tensor scale
        full = np.concatenate([codecs.dequantize_nvfp4(p[2], p[3], p[4], k) for p in parts], axis=0)
        wt = torch.from_numpy(full)
        if device.type == "cuda":
            return LinearWeight("w4", None, None, W4Weight.quantize_device(fmt, wt.to(device)))
        return LinearWeight("w4", None, None, W4Weight.quantize(fmt, wt, device))

    def lin(parts) -> LinearWeight:
        if isinstance(parts[0], tuple) and len(parts[0]) == 6 and parts[0][0] == "w4":
            return lin_w4(parts)
        vals = torch.cat([p[0] for p in parts], dim=0).contiguous()
        if parts[0][1] is None:
            return LinearWeight("dense", vals)
        sc = torch.cat([p[1] for p in parts], dim=0)
        return LinearWeight("fp8", vals, sc.t().contiguous())

    qs, fs = cfg.q_size // tp_size, cfg.ffn // tp_size
    if tp_size <= cfg.n_kv_heads:
        ks = cfg.kv_size // tp_size
        kv_lo, kv_hi = tp_rank * ks, (tp_rank + 1) * ks
    else:
        head = tp_rank * cfg.n_kv_heads // tp_size
        kv_lo, kv_hi = head * hd, (head + 1) * hd
    embed = dense("token_embd.weight")
    layers = []
    for i in range(cfg.n_layers):
        p = f"blk.{i}."
        layers.append(LayerWeights(
            attn_norm=dense(p + "attn_norm.weight"),
            qkv=lin([rows(p + "attn_q.weight", tp_rank * qs, (tp_rank + 1) * qs),
                     rows(p + "attn_k.weight", kv_lo, kv_hi), rows(p + "attn_v.weight", kv_lo, kv_hi)]),
            o=lin([rows(p + "attn_output.weight", 0, cfg.d_model, (tp_rank * qs, (tp_rank + 1) * qs))]),
            mlp_norm=dense(p + "ffn_norm.weight"),
            gate_up=lin([rows(p + "ffn_gate.weight", tp_rank * fs, (tp_rank + 1) * fs),
                         rows(p + "ffn_up.weight", tp_rank * fs, (tp_rank + 1) * fs)]),
            down=lin([rows(p + "ffn_down.weight", 0, cfg.d_model, (tp_rank * fs, (tp_rank + 1) * fs))]),
            **{f: dense(p + n) for n, f in _OPTIONAL_LAYER_VECTORS if p + n in g.tensors}))
    final_norm = dense("output_norm.weight")
    vs = (cfg.vocab + tp_size - 1) // tp_size
    vo = tp_rank * vs if tp_size > 1 else 0
    v_hi = min(cfg.vocab, vo + vs) if tp_size > 1 else cfg.vocab
    if cfg.tie_embeddings:
        head = LinearWeight("dense", embed[vo:v_hi].contiguous())
    else:
        head = lin([rows("output.weight", vo, v_hi)])
    return cfg, LlamaWeights(embed, layers, final_norm, head, vo)


def load_model_gguf(g: G.GgufFile, device, tp_size: int = 1, tp_rank: int = 0, ep_size: int = 1, ep_rank: int = 0,
                    kv_format: Optional[str] = None):
    """(cfg, weights, family) of this rank for any model family a file can carry: the dense decoder (`llama`,
    `gemma4`) through load_llama_gguf, `moe` and `qwen35` through models.family_io."""
    cfg = config_from_gguf(g)
    if cfg.family in ("moe", "qwen35"):
        from . import family_io
        cfg, w = family_io.load_family_gguf(g, device, tp_size, tp_rank, ep_size, ep_rank, kv_format=kv_format)
        return cfg, w, cfg.family
    if ep_size != 1:
        raise G.GgufError("expert parallelism applies to the mixture-of-experts family")
    cfg, w = load_llama_gguf(g, device, tp_size, tp_rank, kv_format=kv_format)
    return cfg, w, cfg.family


def vision_tensor_list(w) -> list:
    """(name, tensor) of every tensor of a vision tower, in file order."""
    out = [("v.patch_embd.weight", w.patch_w.w), ("v.patch_embd.bias", w.patch_b), ("v.position_embd.weight", w.pos_table)]
    for i, b in enumerate(w.blocks):
        p = f"v.blk.{i}."
        out += [(p + "ln1.weight", b.norm1_w), (p + "ln1.bias", b.norm1_b), (p + "ln2.weight", b.norm2_w),
                (p + "ln2.bias", b.norm2_b), (p + "attn_qkv.weight", b.qkv.w), (p + "attn_qkv.bias", b.qkv_b),
                (p + "attn_out.weight", b.proj.w), (p + "attn_out.bias", b.proj_b), (p + "ffn_up.weight", b.fc1.w),
                (p + "ffn_up.bias", b.fc1_b), (p + "ffn_down.weight", b.fc2.w), (p + "ffn_down.bias", b.fc2_b)]
    out += [("v.merger.ln.weight", w.merger_norm_w), ("v.merger.ln.bias", w.merger_norm_b),
            ("v.merger.fc1.weight", w.merger_fc1.w), ("v.merger.fc1.bias", w.merger_fc1_b),
            ("v.merger.fc2.weight", w.merger_fc2.w), ("v.merger.fc2.bias", w.merger_fc2_b)]
    return out


def load_vision_gguf(g: G.GgufFile, cfg: ModelConfig, device):
    """(VisionConfig, VisionWeights) of a verified open GGUF file, or None when it carries no tower."""
    if not cfg.vision or "v.patch_embd.weight" not in g.tensors:
        return None
    from .vision_tower import VisionBlock, VisionConfig, VisionWeights
    vc = VisionConfig(**cfg.vision)
    if vc.out_hidden != cfg.d_model:
        raise G.GgufError("the vision tower's output width differs from the language model's")
    dt = torch.float32 if cfg.weight_format == "fp32" else torch.bfloat16
    want = G.T_F32 if dt == torch.float32 else G.T_BF16

    def t(name):
        e = g.tensors.get(name)
        if e is None:
            raise G.GgufError(f"incomplete vision tower: {name} is missing")
        if e.ttype != want:
            raise G.GgufError(f"{name}: unexpected tensor type {e.ttype}")
        return g.upload(name, torch.device(device), dt).view(e.shape)

    def lw(name):
        return LinearWeight("dense", t(name))
    w = VisionWeights(lw("v.patch_embd.weight"), t("v.patch_embd.bias"), t("v.position_embd.weight"))
    for i in range(vc.depth):
        p = f"v.blk.{i}."
        w.blocks.append(VisionBlock(t(p + "ln1.weight"), t(p + "ln1.bias"), t(p + "ln2.weight"), t(p + "ln2.bias"),
                                    lw(p + "attn_qkv.weight"), t(p + "attn_qkv.bias"), lw(p + "attn_out.weight"),
                                    t(p + "attn_out.bias"), lw(p + "ffn_up.weight"), t(p + "ffn_up.bias"),
                                    lw(p + "ffn_down.weight"), t(p + "ffn_down.bias")))
    w.merger_norm_w, w.merger_norm_b = t("v.merger.ln.weight"), t("v.merger.ln.bias")
    w.merger_fc1, w.merger_fc1_b = lw("v.merger.fc1.weight"), t("v.merger.fc1.bias")
    w.merger_fc2, w.merger_fc2_b = lw("v.merger.fc2.weight"), t("v.merger.fc2.bias")
    return vc, w


def load_mtp_gguf(g: G.GgufFile, cfg: ModelConfig, device):
    """The multi-token-prediction component of a verified open GGUF file (models.mtp.MtpWeights), or None when
    the file carries none.  The component is dense (fp32 with an fp32 model, bf16 otherwise)."""
    if "mtp.fc.weight" not in g.tensors:
        return None
    from .mtp import MtpWeights
    dt = torch.float32 if cfg.weight_format == "fp32" else torch.bfloat16
    want = G.T_F32 if dt == torch.float32 else G.T_BF16

    def dense(name):
        t = g.tensors.get(name)
        if t is None:
            raise G.GgufError(f"incomplete MTP component: {name} is missing")
        if t.ttype != want:
            raise G.GgufError(f"{name}: unexpected tensor type {t.ttype}")
        return g.upload(name, torch.device(device), dt).view(t.shape)

    d = cfg.d_model
    fc = dense("mtp.fc.weight")
    if tuple(fc.shape) != (d, 2 * d):
        raise G.GgufError("mtp.fc.weight must be [d_model, 2 * d_model]")
    p = "mtp.blk.0."
    layer = LayerWeights(attn_norm=dense(p + "attn_norm.weight"), qkv=LinearWeight("dense", dense(p + "attn_qkv.weight")),
                         o=LinearWeight("dense", dense(p + "attn_output.weight")), mlp_norm=dense(p + "ffn_norm.weight"),
                         gate_up=LinearWeight("dense", dense(p + "ffn_gate_up.weight")),
                         down=LinearWeight("dense", dense(p + "ffn_down.weight")))
    return MtpWeights(LinearWeight("dense", fc), dense("mtp.pre_fc_norm_embedding.weight"),
                      dense("mtp.pre_fc_norm_hidden.weight"), layer, dense("mtp.norm.weight"))


def tokenizer_from_gguf(g: G.GgufFile):
    """HF `tokenizers` JSON embedded in the file, or the byte tokenizer when absent."""
    from ..frontend.text import ByteTokenizer, HFTokenizer
    raw = g.metadata.get(G.FRONTEND_TOKENIZER_KEY)
    if raw is None:
        return ByteTokenizer()
    return HFTokenizer(raw)

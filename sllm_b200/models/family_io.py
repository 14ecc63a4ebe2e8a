"""GGUF <-> resident weights for the mixture-of-experts family and the gated-delta-net hybrid family.

Files hold the unsharded model; a rank of a tensor- / expert-parallel run reads only its share: attention and
gated-delta-net projections by head, MLP matrices by intermediate channel, routed experts by expert range, the output
matrix by vocabulary range.  Dense matrices travel as BF16 (F32 for the fp32 check models), routed experts as standard
GGML MXFP4 blocks (type 39; NVFP4 experts as type 40 plus an outer-scale tensor), all experts of a layer in one tensor
whose rows are expert-major.

Tensor names, MoE layer i:  blk.i.attn_norm | attn_q | attn_k | attn_v | attn_output | attn_sinks | ffn_norm |
ffn_gate_inp (router; rows past n_experts: the shared-expert gate and zero padding) | ffn_gate_up_exps | ffn_down_exps |
ffn_gate_up_shexp | ffn_down_shexp.  Hybrid layer i: blk.i.attn_norm | ffn_norm | ffn_gate | ffn_up | ffn_down (or, with
a sparse MLP, the ffn_gate_inp / ffn_*_exps / ffn_*_shexp tensors of the MoE layer) and either
attn_q | attn_k | attn_v | attn_gate | attn_output | attn_q_norm | attn_k_norm (full attention) or ssm_in | ssm_conv1d |
ssm_a | ssm_dt | ssm_norm | ssm_out (gated delta net).

Reference: the per-family conversion plans of crates/sllm-core/src/gguf_convert.rs:145-704 (Qwen3.5 BF16 / FP8 /
MoE-MXFP4 plans) and the expert tensor contract of crates/sllm-core/src/qwen35_moe.rs:1277-1600.
"""
from __future__ import annotations

import json
from typing import Optional

import numpy as np
import torch

from ..formats import codecs
from ..formats import gguf as G
from ..ops.core import LinearWeight
from ..ops.w4 import W4Weight
from .config import ModelConfig
from .loader import CONVERTER_ID, FP8_ENCODING, MXFP4_ENCODING, NVFP4_ENCODING, config_from_gguf

FAMILIES = ("moe", "qwen35")


def _bytes(t: torch.Tensor) -> tuple:
    """(gguf type, payload) of a dense tensor: F32 stays F32, everything else travels as BF16."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.float32:
        return G.T_F32, t.numpy().astype("<f4").tobytes()
    return G.T_BF16, t.to(torch.bfloat16).view(torch.int16).numpy().astype("<i2").tobytes()


class _Sink:
    def __init__(self):
        self.tensors, self.bindings = [], []

    def dense(self, name: str, t: Optional[torch.Tensor]) -> None:
        if t is None:
            return
        ttype, raw = _bytes(t)
        self.tensors.append((name, tuple(t.shape), ttype, raw))

    def linear(self, name: str, lw: Optional[LinearWeight], r0: int = 0, r1: Optional[int] = None) -> None:
        if lw is None:
            return
        r1 = r1 if r1 is not None else lw.w.shape[0]
        if lw.kind == "fp8":
            # E4M3 bytes + the file layout of the 1 x 128 block scales, [N, ceil(K / 128)] fp32
            val = lw.w[r0:r1].detach().cpu().contiguous()
            sc = lw.scale_t[:, r0:r1].t().detach().cpu().float().contiguous()
            self.tensors.append((name, tuple(val.shape), G.T_I8, val.numpy().tobytes()))
            self.tensors.append((name + ".scale", tuple(sc.shape), G.T_F32, sc.numpy().astype("<f4").tobytes()))
            self.bindings.append({"logical_tensor": name, "value_tensor": name, "encoding": FP8_ENCODING, "role": "weight",
                                  "logical_shape": list(val.shape), "scope": "consumed",
                                  "scales": [{"role": "block", "tensor": name + ".scale"}]})
            return
        if lw.kind != "dense":
            raise G.GgufError(f"{name}: this family writes dense or FP8 projections (found {lw.kind})")
        self.dense(name, lw.w[r0:r1])

    def experts(self, name: str, w4: W4Weight) -> None:
        """All groups of a 4-bit weight as one tensor [groups * n, k], expert-major rows."""
        parts = [w4.to_file_layout(g) for g in range(w4.groups)]
        packed = np.concatenate([p[0] for p in parts], axis=0)
        scales = np.concatenate([p[1] for p in parts], axis=0)
        shape = (w4.groups * w4.n, w4.k)
        binding = {"logical_tensor": name, "value_tensor": name, "role": "weight", "logical_shape": list(shape),
                   "scope": "consumed", "scales": []}
        if w4.fmt == "mxfp4":
            self.tensors.append((name, shape, G.T_MXFP4, codecs.to_ggml_mxfp4(packed, scales, w4.k)))
            binding["encoding"] = MXFP4_ENCODING
        else:
            self.tensors.append((name, shape, G.T_NVFP4, codecs.to_ggml_nvfp4(packed, scales, w4.k)))
            ts = w4.tensor_scale.detach().cpu().float().contiguous()
            self.tensors.append((name + ".outer_scale", (w4.groups,), G.T_F32, ts.numpy().astype("<f4").tobytes()))
            binding["encoding"] = NVFP4_ENCODING
            binding["scales"] = [{"role": "outer", "tensor": name + ".outer_scale"}]
        self.bindings.append(binding)


def export_family_gguf(cfg: ModelConfig, w, path: str, tokenizer_json: Optional[str] = None,
                       chat_template: Optional[str] = None, converter_args: Optional[dict] = None,
                       known_unconsumed: Optional[list] = None, source_fingerprints: tuple = ()) -> dict:
    """Writes unsharded weights of a `moe` or `qwen35` model; returns the derived lock document.  `known_unconsumed`
    names source tensors the converter left out on purpose (vision tower, multi-token-prediction head); they are
    recorded in the tensor recipe."""
    if cfg.family not in FAMILIES:
        raise G.GgufError(f"family {cfg.family!r} is written by models.loader.export_llama_gguf")
    s = _Sink()
    s.dense("token_embd.weight", w.embed)
    q, kv, f = cfg.q_size, cfg.kv_size, cfg.ffn
    for i, l in enumerate(w.layers):
        p = f"blk.{i}."
        if cfg.family == "moe":
            s.dense(p + "attn_norm.weight", l.attn_norm)
            s.linear(p + "attn_q.weight", l.qkv, 0, q)
            s.linear(p + "attn_k.weight", l.qkv, q, q + kv)
            s.linear(p + "attn_v.weight", l.qkv, q + kv, q + 2 * kv)
            s.linear(p + "attn_output.weight", l.o)
            s.dense(p + "attn_sinks.weight", l.sinks)
            s.dense(p + "ffn_norm.weight", l.mlp_norm)
            s.linear(p + "ffn_gate_inp.weight", l.router)
            s.experts(p + "ffn_gate_up_exps.weight", l.gate_up)
            s.experts(p + "ffn_down_exps.weight", l.down)
            s.linear(p + "ffn_gate_up_shexp.weight", l.shared_gate_up)
            s.linear(p + "ffn_down_shexp.weight", l.shared_down)
        else:
            s.dense(p + "attn_norm.weight", l.in_norm)
            s.dense(p + "ffn_norm.weight", l.mlp_norm)
            if l.router is not None:
                s.linear(p + "ffn_gate_inp.weight", l.router)
                s.experts(p + "ffn_gate_up_exps.weight", l.exp_gate_up)
                s.experts(p + "ffn_down_exps.weight", l.exp_down)
                s.linear(p + "ffn_gate_up_shexp.weight", l.shared_gate_up)
                s.linear(p + "ffn_down_shexp.weight", l.shared_down)
            else:
                s.linear(p + "ffn_gate.weight", l.gate_up, 0, f)
                s.linear(p + "ffn_up.weight", l.gate_up, f, 2 * f)
                s.linear(p + "ffn_down.weight", l.down)
            if l.kind == "full":
                s.linear(p + "attn_q.weight", l.qkv, 0, q)
                s.linear(p + "attn_k.weight", l.qkv, q, q + kv)
                s.linear(p + "attn_v.weight", l.qkv, q + kv, q + 2 * kv)
                s.linear(p + "attn_gate.weight", l.gate)
                s.linear(p + "attn_output.weight", l.o)
                s.dense(p + "attn_q_norm.weight", l.q_norm)
                s.dense(p + "attn_k_norm.weight", l.k_norm)
            else:
                n_in = _gdn_in_rows(cfg)
                s.linear(p + "ssm_in.weight", l.in_proj, 0, n_in)        # without the padding rows
                s.dense(p + "ssm_conv1d.weight", l.conv_w)
                s.dense(p + "ssm_a", l.a_log)
                s.dense(p + "ssm_dt.bias", l.dt_bias)
                s.dense(p + "ssm_norm.weight", l.out_norm)
                s.linear(p + "ssm_out.weight", l.out_proj)
    s.dense("output_norm.weight", w.final_norm)
    if not cfg.tie_embeddings:
        s.linear("output.weight", w.lm_head)
    md = {"general.architecture": "sllm-" + cfg.family, "general.name": cfg.name,
          G.FRONTEND_CONFIG_KEY: json.dumps(cfg.to_dict(), sort_keys=True)}
    if tokenizer_json is not None:
        md[G.FRONTEND_TOKENIZER_KEY] = tokenizer_json
    if chat_template is not None:
        md["tokenizer.chat_template"] = chat_template
    md.update(G.recipe_metadata(s.bindings, known_unconsumed=known_unconsumed))
    digests = G.write_gguf(path, md, s.tensors)
    return G.make_derived_lock(path, digests, f"{cfg.name}:{cfg.family}", list(source_fingerprints), {"id": CONVERTER_ID, "args": converter_args or {}})


def _gdn_in_rows(cfg: ModelConfig) -> int:
    return (2 * cfg.gdn_qk_heads + cfg.gdn_heads) * cfg.gdn_head_dim + cfg.gdn_heads * cfg.gdn_head_dim + 2 * cfg.gdn_heads


class _Source:
    def __init__(self, g: G.GgufFile, cfg: ModelConfig, device):
        self.g, self.cfg, self.device = g, cfg, torch.device(device)
        self.dt = torch.float32 if cfg.weight_format == "fp32" else torch.bfloat16
        rec = g.recipe() or {"bindings": []}
        self.bound = {b["logical_tensor"]: b for b in rec["bindings"]}

    def has(self, name: str) -> bool:
        return name in self.g.tensors

    def dense(self, name: str, keep_f32: bool = False) -> torch.Tensor:
        t = self.g.tensors[name]
        if t.ttype == G.T_F32:
            v = self.g.upload(name, self.device, torch.float32).view(t.shape)
            return v if (keep_f32 or self.dt == torch.float32) else v.to(self.dt)
        if t.ttype == G.T_BF16:
            v = self.g.upload(name, self.device, torch.bfloat16).view(t.shape)
            return v.float() if keep_f32 else v.to(self.dt) if self.dt != torch.bfloat16 else v
        raise G.GgufError(f"{name}: unexpected tensor type {t.ttype}")

    def head_rows(self, name: str, segments: list, tp_size: int, tp_rank: int, transpose: bool = False,
                  keep_f32: bool = False) -> torch.Tensor:
        """This rank's rows (columns with ``transpose``) of a matrix whose rows are consecutive (heads, rows per head)
        segments, each split evenly by head."""
        w = self.dense(name, keep_f32=keep_f32)
        if tp_size == 1:
            return w
        if transpose:
            w = w.t()
        out, r0 = [], 0
        for heads, per in segments:
            if heads % tp_size:
                raise G.GgufError(f"{name}: {heads} heads do not divide over {tp_size} ranks")
            loc = heads // tp_size
            out.append(w[r0 + tp_rank * loc * per:r0 + (tp_rank + 1) * loc * per])
            r0 += heads * per
        w = torch.cat(out, dim=0)
        return (w.t() if transpose else w).contiguous()

    # ---- projections: bf16 / fp32 values, or E4M3 bytes with [N, ceil(K / 128)] block scales
    def matrix(self, name: str) -> tuple:
        """(values [N, K], block scales [N, ceil(K / 128)] or None)."""
        t = self.g.tensors[name]
        if t.ttype == G.T_I8:
            b = self.bound.get(name)
            if b is None or b["encoding"] != FP8_ENCODING:
                raise G.GgufError(f"{name}: 8-bit tensor without a block-scaled FP8 binding")
            sc_name = [x["tensor"] for x in b.get("scales", []) if x.get("role") == "block"]
            if len(sc_name) != 1:
                raise G.GgufError(f"{name}: an FP8 binding needs exactly one block-scale tensor")
            val = self.g.upload(name, self.device, torch.uint8).view(t.shape)
            sc = self.g.upload(sc_name[0], self.device, torch.float32).view(self.g.tensors[sc_name[0]].shape)
            if sc.shape != (t.shape[0], (t.shape[1] + 127) // 128):
                raise G.GgufError(f"{name}: block-scale tensor shape {tuple(sc.shape)} does not match")
            return val, sc
        return self.dense(name), None

    @staticmethod
    def _segments(n: int, segments: list, tp_size: int, tp_rank: int, what: str) -> list:
        """Index ranges of this rank's share of `n` rows that are consecutive (heads, rows per head) segments."""
        out, r0 = [], 0
        for heads, per in segments:
            if heads % tp_size:
                raise G.GgufError(f"{what}: {heads} heads do not divide over {tp_size} ranks")
            loc = heads // tp_size
            out.append((r0 + tp_rank * loc * per, r0 + (tp_rank + 1) * loc * per))
            r0 += heads * per
        return out

    def shard(self, name: str, segments: list, tp_size: int, tp_rank: int, transpose: bool = False) -> tuple:
        """This rank's rows (columns with `transpose`) of a projection, as `matrix` returns it."""
        val, sc = self.matrix(name)
        if tp_size == 1:
            return val, sc
        if not transpose:
            rs = self._segments(val.shape[0], segments, tp_size, tp_rank, name)
            val = torch.cat([val[a:b] for a, b in rs], dim=0)
            sc = None if sc is None else torch.cat([sc[a:b] for a, b in rs], dim=0)
            return val.contiguous(), sc
        cs = self._segments(val.shape[1], segments, tp_size, tp_rank, name)
        if sc is not None and any(a % 128 or b % 128 for a, b in cs):
            raise G.GgufError(f"{name}: a column shard of a block-scaled FP8 matrix must fall on 128-column borders")
        val = torch.cat([val[:, a:b] for a, b in cs], dim=1)
        sc = None if sc is None else torch.cat([sc[:, a // 128:b // 128] for a, b in cs], dim=1)
        return val.contiguous(), sc

    @staticmethod
    def cat_rows(parts: list, pad_to: int = 1) -> tuple:
        val = torch.cat([p[0] for p in parts], dim=0)
        sc = None if parts[0][1] is None else torch.cat([p[1] for p in parts], dim=0)
        pad = (-val.shape[0]) % pad_to
        if pad:
            val = torch.cat([val, torch.zeros((pad, val.shape[1]), dtype=val.dtype, device=val.device)], dim=0)
            if sc is not None:
                sc = torch.cat([sc, torch.ones((pad, sc.shape[1]), dtype=sc.dtype, device=sc.device)], dim=0)
        return val, sc

    @staticmethod
    def to_linear(m: tuple) -> LinearWeight:
        val, sc = m
        if sc is None:
            return LinearWeight("dense", val.contiguous())
        return LinearWeight("fp8", val.contiguous(), sc.t().contiguous())

    def experts(self, name: str, groups: int, g_lo: int, g_hi: int) -> W4Weight:
        t = self.g.tensors[name]
        b = self.bound.get(name)
        if b is None:
            raise G.GgufError(f"{name}: 4-bit expert tensor without a recipe binding")
        rows, k = t.shape
        if rows % groups:
            raise G.GgufError(f"{name}: {rows} rows do not split into {groups} experts")
        n = rows // groups
        raw = self.g.upload(name, "cpu", torch.uint8).numpy().tobytes()
        if b["encoding"] == MXFP4_ENCODING and t.ttype == G.T_MXFP4:
            fmt, ts = "mxfp4", None
            packed, scales = codecs.from_ggml_mxfp4(raw, rows, k)
        elif b["encoding"] == NVFP4_ENCODING and t.ttype == G.T_NVFP4:
            fmt = "nvfp4"
            outer = [x for x in b.get("scales", []) if x.get("role") == "outer"]
            if len(outer) != 1:
                raise G.GgufError(f"{name}: an NVFP4 binding needs exactly one outer scale")
            ts = self.g.upload(outer[0]["tensor"], "cpu", torch.float32).numpy()[g_lo:g_hi]
            packed, scales = codecs.from_ggml_nvfp4(raw, rows, k)
        else:
            raise G.GgufError(f"{name}: binding {b['encoding']} does not match tensor type {t.ttype}")
        packed = packed.reshape(groups, n, -1)[g_lo:g_hi]
        scales = scales.reshape(groups, n, -1)[g_lo:g_hi]
        return W4Weight.from_file_layout(fmt, np.ascontiguousarray(packed), np.ascontiguousarray(scales), k, ts, self.device)


def load_family_gguf(g: G.GgufFile, device, tp_size: int = 1, tp_rank: int = 0, ep_size: int = 1, ep_rank: int = 0,
                     kv_format: Optional[str] = None):
    """(cfg, weights) of this rank for a `moe` or `qwen35` file."""
    cfg = config_from_gguf(g)
    if cfg.family not in FAMILIES:
        raise G.GgufError(f"family {cfg.family!r} is read by models.loader.load_llama_gguf")
    if kv_format:
        cfg.kv_format = kv_format
    src = _Source(g, cfg, device)
    L = src.to_linear
    d, hd, hq, hkv, f = cfg.d_model, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn
    if hq % tp_size or (hkv % tp_size and tp_size % hkv):
        raise G.GgufError("attention heads do not divide over the tensor-parallel ranks")
    kv_seg = [(hkv, hd)] if tp_size <= hkv else None

    def kv_rows(name):
        if kv_seg is not None:
            return src.shard(name, kv_seg, tp_size, tp_rank)
        head = tp_rank * hkv // tp_size          # fewer kv heads than ranks: the head this rank's query group uses
        val, sc = src.matrix(name)
        return val[head * hd:(head + 1) * hd], None if sc is None else sc[head * hd:(head + 1) * hd]

    def qkv(p):
        return L(src.cat_rows([src.shard(p + "attn_q.weight", [(hq, hd)], tp_size, tp_rank), kv_rows(p + "attn_k.weight"),
                               kv_rows(p + "attn_v.weight")]))

    embed = src.dense("token_embd.weight")
    layers = []
    if cfg.family == "moe":
        from .moe import MoeLayerWeights, MoeWeights
        if cfg.n_experts % ep_size:
            raise G.GgufError("experts do not divide over the expert-parallel ranks")
        per = cfg.n_experts // ep_size
        e_lo, e_hi = ep_rank * per, (ep_rank + 1) * per
        for i in range(cfg.n_layers):
            p = f"blk.{i}."
            sinks = None
            if src.has(p + "attn_sinks.weight"):
                sinks = src.dense(p + "attn_sinks.weight", keep_f32=True)
                sinks = sinks[tp_rank * (hq // tp_size):(tp_rank + 1) * (hq // tp_size)].contiguous()
            shared = {}
            if src.has(p + "ffn_gate_up_shexp.weight"):
                shared = dict(shared_gate_up=L(src.matrix(p + "ffn_gate_up_shexp.weight")),
                              shared_down=L(src.matrix(p + "ffn_down_shexp.weight")))
            layers.append(MoeLayerWeights(
                attn_norm=src.dense(p + "attn_norm.weight"), qkv=qkv(p),
                o=L(src.shard(p + "attn_output.weight", [(hq, hd)], tp_size, tp_rank, transpose=True)),
                sinks=sinks, mlp_norm=src.dense(p + "ffn_norm.weight"), router=L(src.matrix(p + "ffn_gate_inp.weight")),
                gate_up=src.experts(p + "ffn_gate_up_exps.weight", cfg.n_experts, e_lo, e_hi),
                down=src.experts(p + "ffn_down_exps.weight", cfg.n_experts, e_lo, e_hi), **shared))
        make = MoeWeights
    else:
        from .qwen35 import Qwen35Layer, Qwen35Weights
        ghd, vh, qh = cfg.gdn_head_dim, cfg.gdn_heads, cfg.gdn_qk_heads
        sparse = cfg.n_experts > 0
        for name, v in (("gdn_heads", vh), ("gdn_qk_heads", qh), ("ffn", tp_size if sparse else f)):
            if v % tp_size:
                raise G.GgufError(f"{name} = {v} does not divide over {tp_size} tensor-parallel ranks")
        if sparse and cfg.n_experts % ep_size:
            raise G.GgufError("experts do not divide over the expert-parallel ranks")
        per = cfg.n_experts // ep_size if sparse else 0
        e_lo, e_hi = ep_rank * per, (ep_rank + 1) * per
        norm_dt = torch.bfloat16 if src.dt != torch.float32 else torch.float32
        for i in range(cfg.n_layers):
            p = f"blk.{i}."
            common = dict(in_norm=src.dense(p + "attn_norm.weight"), mlp_norm=src.dense(p + "ffn_norm.weight"))
            if sparse:
                common.update(router=L(src.matrix(p + "ffn_gate_inp.weight")),
                              exp_gate_up=src.experts(p + "ffn_gate_up_exps.weight", cfg.n_experts, e_lo, e_hi),
                              exp_down=src.experts(p + "ffn_down_exps.weight", cfg.n_experts, e_lo, e_hi))
                if src.has(p + "ffn_gate_up_shexp.weight"):
                    common.update(shared_gate_up=L(src.matrix(p + "ffn_gate_up_shexp.weight")),
                                  shared_down=L(src.matrix(p + "ffn_down_shexp.weight")))
            else:
                gate_up = src.cat_rows([src.shard(p + "ffn_gate.weight", [(f, 1)], tp_size, tp_rank),
                                        src.shard(p + "ffn_up.weight", [(f, 1)], tp_size, tp_rank)])
                common.update(gate_up=L(gate_up),
                              down=L(src.shard(p + "ffn_down.weight", [(f, 1)], tp_size, tp_rank, transpose=True)))
            if (i + 1) % cfg.full_attention_interval == 0:
                gate = None
                if src.has(p + "attn_gate.weight"):
                    gate = L(src.shard(p + "attn_gate.weight", [(hq, hd)], tp_size, tp_rank))
                layers.append(Qwen35Layer("full", qkv=qkv(p), gate=gate,
                                          o=L(src.shard(p + "attn_output.weight", [(hq, hd)], tp_size, tp_rank, transpose=True)),
                                          q_norm=src.dense(p + "attn_q_norm.weight").to(norm_dt),
                                          k_norm=src.dense(p + "attn_k_norm.weight").to(norm_dt), **common))
            else:
                segs = [(qh, ghd), (qh, ghd), (vh, ghd), (vh, ghd), (vh, 1), (vh, 1)]
                w_in = src.cat_rows([src.shard(p + "ssm_in.weight", segs, tp_size, tp_rank)], pad_to=8)
                layers.append(Qwen35Layer(
                    "gdn", in_proj=L(w_in), conv_w=src.head_rows(p + "ssm_conv1d.weight", segs[:3], tp_size, tp_rank),
                    a_log=src.head_rows(p + "ssm_a", [(vh, 1)], tp_size, tp_rank, keep_f32=True).contiguous(),
                    dt_bias=src.head_rows(p + "ssm_dt.bias", [(vh, 1)], tp_size, tp_rank),
                    out_norm=src.dense(p + "ssm_norm.weight", keep_f32=True),
                    out_proj=L(src.shard(p + "ssm_out.weight", [(vh, ghd)], tp_size, tp_rank, transpose=True)), **common))
        make = Qwen35Weights
    final_norm = src.dense("output_norm.weight")
    vs = (cfg.vocab + tp_size - 1) // tp_size
    vo = tp_rank * vs if tp_size > 1 else 0
    v_hi = min(cfg.vocab, vo + vs) if tp_size > 1 else cfg.vocab
    if tp_size == 1 and cfg.tie_embeddings:
        head = LinearWeight("dense", embed)
    elif cfg.tie_embeddings:
        head = LinearWeight("dense", embed[vo:v_hi].contiguous())
    else:
        val, sc = src.matrix("output.weight")
        head = L((val[vo:v_hi], None if sc is None else sc[vo:v_hi]))
    return cfg, make(embed, layers, final_norm, head, vo)

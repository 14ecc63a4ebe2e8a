"""Llama-style dense decoder (RMSNorm, split-half RoPE, GQA, SwiGLU) on the op layer.

Per-layer op order follows the reference's dense full-attention layer
(crates/sllm-core/src/qwen_graph.rs:2524-3501: input norm -> q/k/v matmul -> rotary + KV append ->
causal attention -> o matmul -> residual -> post-attention norm -> gate/up matmul -> silu-mul ->
down matmul -> residual; final norm -> lm head -> argmax), with these fusions: q/k/v and gate/up are
single GEMMs, the norms and the activation emit the FP8 operand of the following GEMM, attention
emits the FP8 operand of the o projection, and residual adds live in the GEMM epilogues.

Tensor parallelism (absent from the reference) shards heads and the FFN dimension; the row-parallel
projections (o, down) go through ``tp.row_linear`` which is either the fused GEMM+all-reduce kernel
or the unfused NCCL baseline.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import ops
from ..engine.batch import ForwardBatch
from ..ops import w4 as _w4
from ..ops.core import LinearWeight, QTensor
from .config import ModelConfig


class NoTP:
    """Single-GPU stand-in for the tensor-parallel context."""
    size = 1
    rank = 0

    def row_linear(self, x, w: LinearWeight, residual):
        return ops.linear(x, w, residual)

    def gather_logits(self, logits: torch.Tensor) -> torch.Tensor:
        return logits

    def argmax(self, logits: torch.Tensor, vocab_offset: int) -> torch.Tensor:
        return ops.argmax(logits)


@dataclass
class LayerWeights:
    attn_norm: torch.Tensor
    qkv: LinearWeight
    o: LinearWeight
    mlp_norm: torch.Tensor
    gate_up: LinearWeight
    down: LinearWeight
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    post_attn_norm: Optional[torch.Tensor] = None     # Gemma-style norms applied to the block output before the add
    post_mlp_norm: Optional[torch.Tensor] = None
    layer_scalar: Optional[torch.Tensor] = None       # [1]: multiplies the residual stream at the end of the layer
    _scalar: Optional[float] = None

    def layer_scalar_value(self) -> float:
        if self._scalar is None:        # read once: the value is a launch argument of the scaling kernel
            self._scalar = float(self.layer_scalar.float().item())
        return self._scalar


@dataclass
class LlamaWeights:
    embed: torch.Tensor
    layers: list
    final_norm: torch.Tensor
    lm_head: LinearWeight
    vocab_offset: int = 0


def _randn(shape, std, gen, device, dtype):
    return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)


def _shard_rows(w: torch.Tensor, parts: list, tp_size: int, tp_rank: int) -> torch.Tensor:
    """Row-shard a [sum(parts), K] weight whose row blocks (e.g. q | k | v) are each split across ranks."""
    if tp_size == 1:
        return w
    out, r0 = [], 0
    for p in parts:
        blk = w[r0:r0 + p]
        sz = p // tp_size
        out.append(blk[tp_rank * sz:(tp_rank + 1) * sz])
        r0 += p
    return torch.cat(out, dim=0).contiguous()


def init_random_weights(cfg: ModelConfig, device, seed: int = 0, tp_size: int = 1, tp_rank: int = 0,
                        std: float = 0.02) -> LlamaWeights:
    """Seeded ~N(0, std) weights of the configured shape, quantised to the resident format.

    Every rank draws the full tensor from the same generator and keeps its shard, so a TP run holds
    exactly the weights of the single-GPU run.
    """
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    wf = cfg.weight_format
    dense_dtype = torch.float32 if wf == "fp32" else torch.bfloat16
    kind = "fp8" if wf == "fp8" else "dense"
    d, hd = cfg.d_model, cfg.head_dim
    if cfg.n_kv_heads % tp_size and tp_size % cfg.n_kv_heads:
        raise ValueError("kv heads and tensor-parallel size must divide one another")
    if cfg.n_heads % tp_size or cfg.ffn % tp_size:
        raise ValueError("heads and ffn must be divisible by the tensor-parallel size")

    def lin(w: torch.Tensor) -> LinearWeight:
        if wf in ("nvfp4", "mxfp4"):
            from ..ops.w4 import W4Weight
            return LinearWeight("w4", None, None, W4Weight.quantize_device(wf, w.contiguous()))
        if kind == "fp8":
            q = ops.quant_fp8(w.contiguous())
            return LinearWeight("fp8", q.data, q.scale)
        return LinearWeight("dense", w.contiguous())

    def kv_shard(w_kv: torch.Tensor) -> torch.Tensor:
        # fewer kv heads than ranks: each rank keeps the head its query group uses
        if tp_size <= cfg.n_kv_heads:
            sz = cfg.kv_size // tp_size
            return w_kv[tp_rank * sz:(tp_rank + 1) * sz]
        head = tp_rank * cfg.n_kv_heads // tp_size
        return w_kv[head * hd:(head + 1) * hd]

    embed = _randn((cfg.vocab, d), std, gen, device, dense_dtype)
    layers = []
    for _ in range(cfg.n_layers):
        wq = _randn((cfg.q_size, d), std, gen, device, dense_dtype)
        wk = _randn((cfg.kv_size, d), std, gen, device, dense_dtype)
        wv = _randn((cfg.kv_size, d), std, gen, device, dense_dtype)
        wo = _randn((d, cfg.q_size), std, gen, device, dense_dtype)
        wg = _randn((cfg.ffn, d), std, gen, device, dense_dtype)
        wu = _randn((cfg.ffn, d), std, gen, device, dense_dtype)
        wd = _randn((d, cfg.ffn), std, gen, device, dense_dtype)
        if tp_size > 1:
            qs, fs = cfg.q_size // tp_size, cfg.ffn // tp_size
            wq = wq[tp_rank * qs:(tp_rank + 1) * qs]
            wk, wv = kv_shard(wk), kv_shard(wv)
            wo = wo[:, tp_rank * qs:(tp_rank + 1) * qs]
            wg, wu = wg[tp_rank * fs:(tp_rank + 1) * fs], wu[tp_rank * fs:(tp_rank + 1) * fs]
            wd = wd[:, tp_rank * fs:(tp_rank + 1) * fs]
        if cfg.k_equals_v_full and cfg.layer_window(len(layers)) == 0:
            wv = wk            # no value projection: the value rows of the fused matrix repeat the key rows
        layers.append(LayerWeights(
            layer_scalar=torch.ones(1, device=device, dtype=dense_dtype) if cfg.layer_scalar else None,
            attn_norm=torch.ones(d, device=device, dtype=dense_dtype),
            qkv=lin(torch.cat([wq, wk, wv], dim=0)),
            o=lin(wo),
            mlp_norm=torch.ones(d, device=device, dtype=dense_dtype),
            gate_up=lin(torch.cat([wg, wu], dim=0)),
            down=lin(wd),
            q_norm=torch.ones(hd, device=device, dtype=dense_dtype) if cfg.qk_norm else None,
            k_norm=torch.ones(hd, device=device, dtype=dense_dtype) if cfg.qk_norm else None,
            post_attn_norm=torch.ones(d, device=device, dtype=dense_dtype) if cfg.post_norms else None,
            post_mlp_norm=torch.ones(d, device=device, dtype=dense_dtype) if cfg.post_norms else None))
        del wq, wk, wv, wo, wg, wu, wd
    final_norm = torch.ones(d, device=device, dtype=dense_dtype)
    if cfg.tie_embeddings:
        head = embed
    else:
        head = _randn((cfg.vocab, d), std, gen, device, dense_dtype)
    vocab_offset = 0
    if tp_size > 1:
        vs = (cfg.vocab + tp_size - 1) // tp_size
        vocab_offset = tp_rank * vs
        head = head[vocab_offset:min(cfg.vocab, vocab_offset + vs)]
    return LlamaWeights(embed, layers, final_norm, lin(head), vocab_offset)


class LlamaModel:
    """Stateless forward over a ForwardBatch; KV state lives in the PagedKVCache passed in."""

    def __init__(self, cfg: ModelConfig, weights: LlamaWeights, tp=None):
        self.cfg = cfg
        self.w = weights
        self.tp = tp or NoTP()
        t = self.tp.size
        self.hq = cfg.n_heads // t
        self.hkv = max(1, cfg.n_kv_heads // t)
        self.quant = cfg.weight_format == "fp8"
        self.adapters = None      # models.adapters.AdapterSet applied to every forward while set
        self._fused: dict = {}    # row count -> FusedLlamaDecoder (decode steps of up to 32 rows)
        self._fused_reason = None

    def _fused_decoder(self, b: ForwardBatch):
        """The fused decode chain for this batch, or None when the batch or the model is not covered (prefill rows,
        input embeddings, multi-axis rotary positions, adapters, more than 32 rows)."""
        if not b.tokens.is_cuda or b.logit_rows is not None or b.embeds is not None or b.rope_pos3 is not None:
            return None
        rows = b.num_tokens
        if self._fused_reason is None:
            from . import fused_llama
            self._fused_reason = fused_llama.eligible(self) or ""
        if self._fused_reason:
            return None
        if rows > 32 or (self.adapters is not None and (self.adapters.loras or self.adapters.cvs)):
            # a decode-shaped batch of a model that has the fused chain, on the per-op path
            from ..ops import _lib
            _lib.note_fallback("decode_per_op:rows_above_32" if rows > 32 else "decode_per_op:adapters")
            return None
        dec = self._fused.get(rows)
        if dec is None:
            from .fused_llama import FusedLlamaDecoder
            dec = FusedLlamaDecoder(self, rows, b.tokens.device)
            self._fused[rows] = dec
        return dec

    def _fused_logits(self, dec, b: ForwardBatch, cache) -> torch.Tensor:
        lg = dec.run(b, cache)
        self.last_hidden = dec.h
        return lg

    @property
    def local_kv_heads(self) -> int:
        return self.hkv

    def _norm_in(self, h, norm_w, consumer: LinearWeight, quant_fp8: bool):
        """The RMS-normalised residual stream in the form its consumer takes: FP8 + scales, bf16, or - for a 4-bit
        matrix on the W4A4 path - 4-bit codes, the norm computed inside the quantiser."""
        cfg = self.cfg
        if (consumer.kind == "w4" and _w4.w4a4_enabled() and h.dtype == torch.bfloat16 and norm_w.dtype == torch.bfloat16
                and h.shape[1] % 8 == 0 and h.shape[0] <= _w4.W4A4_MAX_DENSE_ROWS):
            q = _w4.act_quant_fp4(h, consumer.w4.fmt, norm=(norm_w, cfg.rms_eps, cfg.norm_offset_one))
            return _w4.Fp4Act(*q, k=h.shape[1], fmt=consumer.w4.fmt)
        return ops.rmsnorm(h, norm_w, cfg.rms_eps, cfg.norm_offset_one, quant=quant_fp8)

    def hidden(self, b: ForwardBatch, cache) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        hd = cfg.head_dim
        h = b.embeds if b.embeds is not None else ops.embedding(w.embed, b.tokens, cfg.embedding_scale)
        for li, lw in enumerate(w.layers):
            # activations are quantised for the projections that hold FP8 weights (a mixed-precision model has FP8
            # attention and 4-bit MLP matrices)
            q_attn, q_o, q_mlp, q_down = (x.kind == "fp8" for x in (lw.qkv, lw.o, lw.gate_up, lw.down))
            qo = q_o and hd == 128 and h.is_cuda
            kv = cache.layer(li)
            ad = self.adapters
            if ad is not None and (ad.loras or ad.cvs):
                h = self._adapter_layer(li, lw, h, b, kv, ad)
                continue
            x = self._norm_in(h, lw.attn_norm, lw.qkv, q_attn)
            qkv = ops.linear(x, lw.qkv)
            if cfg.qk_norm or cfg.v_norm:
                from ..ops import gdn as _g
                qkv = _g.qk_headnorm(qkv, self.hq, self.hkv, hd, lw.q_norm, lw.k_norm, cfg.rms_eps, cfg.norm_offset_one,
                                     norm_v=cfg.v_norm)
            theta, rdim, poff = cfg.layer_rope(li)
            q = ops.rope_kv_append(qkv, b.positions, b.seq_index, b.block_table, kv, self.hq, self.hkv, hd,
                                   theta, rdim, rope_pos3=b.rope_pos3, mrope_sections=cfg.mrope_sections,
                                   pair_offset=poff)
            a = ops.attention(q, kv, b, self.hq, self.hkv, hd, window=cfg.layer_window(li), quant_out=qo,
                              qkv=qkv, sm_scale=cfg.attn_scale)
            if q_o and not qo:
                a = ops.quant_fp8(a)
            if cfg.post_norms:
                # sandwich norms: the block output is normalised before it joins the residual stream
                o = ops.rmsnorm(self.tp.row_linear(a, lw.o, None), lw.post_attn_norm, cfg.rms_eps, cfg.norm_offset_one)
                h = ops.elementwise("add", h, o)
            else:
                h = self.tp.row_linear(a, lw.o, h)
            x = self._norm_in(h, lw.mlp_norm, lw.gate_up, q_mlp)
            gu = ops.linear(x, lw.gate_up)
            if (lw.down.kind == "w4" and _w4.w4a4_enabled() and gu.dtype == torch.bfloat16
                    and gu.shape[0] <= _w4.W4A4_MAX_DENSE_ROWS):
                # 4-bit activations: SiLU*up runs inside the quantiser of the down projection
                wd = lw.down.w4
                act = _w4.Fp4Act(*_w4.act_quant_fp4(gu, wd.fmt, gated=cfg.act), k=gu.shape[1] // 2, fmt=wd.fmt)
            else:
                act = ops.gated_act(gu, cfg.act, quant=q_down)
            if cfg.post_norms:
                o = ops.rmsnorm(self.tp.row_linear(act, lw.down, None), lw.post_mlp_norm, cfg.rms_eps, cfg.norm_offset_one)
                h = ops.elementwise("add", h, o)
            else:
                h = self.tp.row_linear(act, lw.down, h)
            if lw.layer_scalar is not None:
                h = ops.elementwise("scalar_mul", h, s=lw.layer_scalar_value())
        return h

    def _adapter_layer(self, li, lw, h, b, kv, ad):
        """One layer with LoRA deltas on the projections and the control vector on the residual stream.  The
        projections take bf16 inputs here (the delta needs the unquantised activation); single GPU only."""
        cfg = self.cfg
        hd = cfg.head_dim
        if self.tp.size != 1:
            raise ValueError("adapters are supported without tensor parallelism")
        x = ops.rmsnorm(h, lw.attn_norm, cfg.rms_eps, cfg.norm_offset_one)
        qkv = ad.lora_delta(li, "qkv", x, ops.linear(x, lw.qkv))
        q = ops.rope_kv_append(qkv, b.positions, b.seq_index, b.block_table, kv, self.hq, self.hkv, hd, cfg.rope_theta,
                               cfg.rotary_dim, rope_pos3=b.rope_pos3, mrope_sections=cfg.mrope_sections)
        a = ops.attention(q, kv, b, self.hq, self.hkv, hd, window=cfg.layer_window(li), qkv=qkv)
        h = ad.lora_delta(li, "o", a, ops.linear(a, lw.o, h))
        x = ops.rmsnorm(h, lw.mlp_norm, cfg.rms_eps, cfg.norm_offset_one)
        gu = ad.lora_delta(li, "gate_up", x, ops.linear(x, lw.gate_up))
        act = ops.gated_act(gu, cfg.act)
        h = ad.lora_delta(li, "down", act, ops.linear(act, lw.down, h))
        return ad.control(li, h)

    def _keep(self, h: torch.Tensor) -> torch.Tensor:
        """Remembers the residual stream of the last forward (all rows, before the final norm) for consumers such
        as a multi-token-prediction head; a reference, not a copy."""
        self.last_hidden = h
        return h

    def logits(self, h: torch.Tensor, b: ForwardBatch) -> torch.Tensor:
        """Local (vocab-shard) logits of the requested rows."""
        cfg, w = self.cfg, self.w
        if b.logit_rows is not None:
            h = h.index_select(0, b.logit_rows)
        x = ops.rmsnorm(h, w.final_norm, cfg.rms_eps, cfg.norm_offset_one, quant=w.lm_head.kind == "fp8")
        lg = ops.linear(x, w.lm_head)
        if cfg.logit_softcap > 0:
            lg = ops.elementwise("tanh_softcap", lg, s=cfg.logit_softcap)
        return lg

    def forward(self, b: ForwardBatch, cache) -> torch.Tensor:
        """Full-vocabulary logits [rows, vocab]."""
        dec = self._fused_decoder(b)
        if dec is not None:
            return self.tp.gather_logits(self._fused_logits(dec, b, cache))
        return self.tp.gather_logits(self.logits(self._keep(self.hidden(b, cache)), b))

    def greedy(self, b: ForwardBatch, cache) -> torch.Tensor:
        """Greedy next tokens (int32 [rows]) without materialising gathered logits."""
        dec = self._fused_decoder(b)
        if dec is not None:
            return self.tp.argmax(self._fused_logits(dec, b, cache), self.w.vocab_offset)
        return self.tp.argmax(self.logits(self._keep(self.hidden(b, cache)), b), self.w.vocab_offset)

"""Decode steps of the Llama family through the fused decode kernel: two launches per layer.

A decode step (1..32 rows, block-scaled FP8 weights, head_dim 128) becomes

    embed+quant | [q/k/v + RoPE + KV append] | attention(0) |
    [o-proj + residual + quant | gate/up + SiLU*up + quant | down + residual + quant | q/k/v(l+1) + RoPE + KV append]
    | attention(l+1) | ... | [o | gate/up | down | lm-head] | argmax

where every [...] is ONE persistent kernel (csrc/decode_fused.cu) whose phases hand their outputs to each other
through L2, and attention is the tensor-core paged decode kernel.  RMSNorm never runs as an op: its weight vectors
are folded into the following weight matrices once (`fold_norms`), and the per-row factor is applied by the
consuming phase from the sums of squares the producing phase wrote.

The reference executes the same layer as ~12 kernels (crates/sllm-core/src/qwen_graph.rs:2524-3501).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import ops
from ..ops import fused_decode as fd
from ..ops.core import LinearWeight, QTensor


def _fold(lw: LinearWeight, g: torch.Tensor) -> LinearWeight:
    """W' = W diag(g): the norm weight moves into the columns of the matrix that consumes the normalised row."""
    w = lw.dequantized().to(torch.float32) * g.to(torch.float32).unsqueeze(0)
    if lw.kind == "fp8":
        q = ops.quant_fp8(w.to(torch.bfloat16).contiguous()) if w.is_cuda else QTensor(*ops.reference.quant_fp8_1x128(w))
        return LinearWeight("fp8", q.data, q.scale)
    return LinearWeight(lw.kind, w.to(lw.w.dtype))


def fold_norms(cfg, weights) -> None:
    """Folds every pre-GEMM RMSNorm weight vector into its consumer (q/k/v, gate/up, lm head) and resets the
    vectors to the identity, in place.  A no-op for identity norms (random-init models)."""
    if getattr(weights, "norms_folded", False):
        return
    ident = 0.0 if cfg.norm_offset_one else 1.0

    def eff(v):
        return 1.0 + v.to(torch.float32) if cfg.norm_offset_one else v.to(torch.float32)

    def is_ident(v):
        return bool((v.to(torch.float32) == ident).all().item())

    for lw in weights.layers:
        if not is_ident(lw.attn_norm):
            lw.qkv = _fold(lw.qkv, eff(lw.attn_norm))
            lw.attn_norm.fill_(ident)
        if not is_ident(lw.mlp_norm):
            lw.gate_up = _fold(lw.gate_up, eff(lw.mlp_norm))
            lw.mlp_norm.fill_(ident)
    if not is_ident(weights.final_norm):
        if weights.lm_head.w is weights.embed:
            raise ValueError("a tied output matrix cannot absorb the final norm")
        weights.lm_head = _fold(weights.lm_head, eff(weights.final_norm))
        weights.final_norm.fill_(ident)
    weights.norms_folded = True


def eligible(model) -> Optional[str]:
    """None when the model can take the fused decode path, else the reason it cannot."""
    cfg = model.cfg
    if os.environ.get("SLLM_FUSED_DECODE", "1") == "0":
        return "disabled by SLLM_FUSED_DECODE=0"
    if cfg.weight_format != "fp8":
        return "weights are not block-scaled FP8"
    if cfg.kv_format not in ("bf16", "fp8", "fp8-static"):
        return "KV-cache format not covered by the fused rotary epilogue"
    if cfg.head_dim != 128 or cfg.qk_norm or cfg.post_norms or cfg.mrope_sections:
        return "head_dim / q-k norm / sandwich norms / multi-axis rotary not covered"
    if cfg.v_norm or cfg.layer_scalar or cfg.attn_scale is not None or cfg.rope_proportional or cfg.rope_theta_local:
        return "Gemma-4 attention options not covered"
    if (cfg.rotary_dim or cfg.head_dim) not in (32, 64, 128) or cfg.act not in ("silu", "gelu_tanh"):
        return "rotary width or activation not covered"
    hq, hkv = model.hq, model.hkv
    if cfg.d_model % 128 or (cfg.ffn // model.tp.size) % 128:
        return "model width not a multiple of 128"
    if cfg.tie_embeddings:
        return "tied embeddings"
    if model.tp.size > 1 and getattr(model.tp, "impl", "") != "fused":
        return "tensor parallelism without the fused communicator"
    w0 = model.w.layers[0]
    if any(lw.kind != "fp8" for lw in (w0.qkv, w0.o, w0.gate_up, w0.down, model.w.lm_head)):
        return "a projection is not FP8"
    return None


class FusedLlamaDecoder:
    """Static buffers and the launch chain for one row count."""

    def __init__(self, model, rows: int, device: torch.device):
        cfg = model.cfg
        self.model, self.rows, self.device = model, rows, device
        self.bn = 16 if rows <= 16 else 32
        d, bn = cfg.d_model, self.bn
        self.q_size = model.hq * cfg.head_dim
        self.ffn_local = model.w.layers[0].down.in_features
        z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=device)
        self.h = z((rows, d), torch.bfloat16)
        self.hq, self.hs, self.ssq = z((rows, d), torch.uint8), z((d // 128, bn), torch.float32), z((d // 128, bn), torch.float32)
        self.q = z((rows, self.q_size), torch.bfloat16)
        self.aq, self.a_s = z((rows, self.q_size), torch.uint8), z((self.q_size // 128, bn), torch.float32)
        self.actq = z((rows, self.ffn_local), torch.uint8)
        self.acts = z((self.ffn_local // 128, bn), torch.float32)
        self.vocab_local = model.w.lm_head.out_features
        self.logits = z((rows, self.vocab_local), torch.bfloat16)
        fold_norms(cfg, model.w)
        self.impl = fd.backend()
        # the cluster GEMM's SiLU epilogue reads gate and up rows of the same features from one 128-row tile
        if self.impl == "cluster" and getattr(model.w, "gate_up_interleaved", None) is None:
            model.w.gate_up_interleaved = [fd.interleave_gate_up(lw.gate_up.w, lw.gate_up.scale_t, self.ffn_local)
                                           for lw in model.w.layers]

    # ---- phases
    def _qkv(self, lw, kv, b):
        cfg, m = self.model.cfg, self.model
        ph = fd.phase(fd.ROPE_KV, lw.qkv.w, lw.qkv.scale_t, self.hq, self.hs, n=lw.qkv.out_features, k=cfg.d_model,
                      ssq_in=self.ssq, norm_dim=cfg.d_model, eps=cfg.rms_eps, y=self.q, ldy=self.q_size,
                      ld_s_out=self.bn)
        rope = fd.rope_desc(b.positions, b.seq_index, b.block_table, kv, m.hq, m.hkv, cfg.rotary_dim or cfg.head_dim,
                            cfg.rope_theta)
        return ph, rope

    def _o(self, lw):
        d = self.model.cfg.d_model
        return fd.phase(fd.RESID_QUANT, lw.o.w, lw.o.scale_t, self.aq, self.a_s, n=d, k=self.q_size, y=self.h, ldy=d,
                        residual=self.h, q_out=self.hq, s_out=self.hs, ssq_out=self.ssq, ld_s_out=self.bn)

    def _gate_up(self, lw):
        cfg = self.model.cfg
        return fd.phase(fd.SILU_QUANT, lw.gate_up.w, lw.gate_up.scale_t, self.hq, self.hs, n=self.ffn_local,
                        k=cfg.d_model, dual_off=self.ffn_local, ssq_in=self.ssq, norm_dim=cfg.d_model, eps=cfg.rms_eps,
                        act=0 if cfg.act == "silu" else 1, q_out=self.actq, s_out=self.acts, ld_s_out=self.bn)

    def _down(self, lw):
        d = self.model.cfg.d_model
        return fd.phase(fd.RESID_QUANT, lw.down.w, lw.down.scale_t, self.actq, self.acts, n=d, k=self.ffn_local,
                        y=self.h, ldy=d, residual=self.h, q_out=self.hq, s_out=self.hs, ssq_out=self.ssq,
                        ld_s_out=self.bn)

    def _head(self):
        cfg, w = self.model.cfg, self.model.w
        return fd.phase(fd.PLAIN, w.lm_head.w, w.lm_head.scale_t, self.hq, self.hs, n=self.vocab_local, k=cfg.d_model,
                        ssq_in=self.ssq, norm_dim=cfg.d_model, eps=cfg.rms_eps, y=self.logits, ldy=self.vocab_local,
                        softcap=cfg.logit_softcap, ld_s_out=self.bn)

    def run(self, b, cache) -> torch.Tensor:
        """Local logits [rows, vocab shard] (bf16); the final residual stream stays in ``self.h``."""
        m, cfg = self.model, self.model.cfg
        w, rows, dev = m.w, self.rows, self.device
        # the persistent kernel numbers its exchange slots per tile, the cluster GEMM per (tile, K slice): two regions
        comm = None if m.tp.size == 1 else (m.tp.desc if self.impl == "cluster" else m.tp.desc_fd)
        fd.embed_quant(w.embed, b.tokens, self.h, self.hq, self.hs, self.ssq, cfg.embedding_scale)
        ph, rope = self._qkv(w.layers[0], cache.layer(0), b)
        fd.launch([ph], rows, dev, rope, impl=self.impl)
        out = QTensor(self.aq, self.a_s)
        n_layers = len(w.layers)
        for li, lw in enumerate(w.layers):
            phases = [self._o(lw), self._gate_up(lw), self._down(lw)]
            ops.paged_attention(self.q, cache.layer(li), b.block_table, b.seq_index, b.kv_lens, m.hq, m.hkv,
                                cfg.head_dim, window=cfg.layer_window(li), max_kv=b.max_kv, quant_out=True, out=out)
            rope = None
            if li + 1 < n_layers:
                ph, rope = self._qkv(w.layers[li + 1], cache.layer(li + 1), b)
                phases.append(ph)
            else:
                phases.append(self._head())
            il = [None, w.gate_up_interleaved[li], None, None] if self.impl == "cluster" else None
            fd.launch(phases, rows, dev, rope, comm=comm, impl=self.impl, interleaved=il)
        return self.logits

"""Sparse mixture-of-experts decoder (gpt-oss-class shape): GQA attention with per-head sink logits and
alternating sliding-window / full layers, a bf16 router with top-k selection, MXFP4 experts with a gated MLP.

Attention and router run in bf16; expert weights stay MXFP4 (E2M1 codes + E8M0 scales per 32 elements) and go
through the grouped W4A16 tcgen05 GEMM.  With expert parallelism each rank holds n_experts / ep experts and the
attention is tensor-parallel over the same ranks (reference counterpart: the Qwen3.5 MoE graph,
crates/sllm-core/src/qwen35_moe.rs, moe.rs routing contract; single GPU there).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..engine.batch import ForwardBatch
from ..ops import moe as M
from ..ops.core import LinearWeight
from ..ops.w4 import W4Weight
from ..parallel.ep import NoEP
from .config import ModelConfig
from .llama import NoTP, _randn


@dataclass
class MoeLayerWeights:
    attn_norm: torch.Tensor
    qkv: LinearWeight
    o: LinearWeight
    sinks: Optional[torch.Tensor]      # fp32 [local q heads]
    mlp_norm: torch.Tensor
    router: LinearWeight               # [E, d] bf16
    gate_up: W4Weight                  # local experts, [2 * expert_ffn, d] each
    down: W4Weight                     # local experts, [d, expert_ffn] each
    # always-on shared expert (Qwen3.5 MoE): dense gated MLP whose output joins the routed sum under a per-token
    # sigmoid gate; the gate vector rides as row n_experts of `router` (rows above it are zero padding)
    shared_gate_up: Optional[LinearWeight] = None     # [2 * shared_expert_ffn, d]
    shared_down: Optional[LinearWeight] = None        # [d, shared_expert_ffn]


@dataclass
class MoeWeights:
    embed: torch.Tensor
    layers: list
    final_norm: torch.Tensor
    lm_head: LinearWeight
    vocab_offset: int = 0


def init_random_moe_weights(cfg: ModelConfig, device, seed: int = 0, tp_size: int = 1, tp_rank: int = 0,
                            ep_size: int = 1, ep_rank: int = 0, std: float = 0.02) -> MoeWeights:
    """Seeded random weights; every rank draws the same tensors and keeps its shard (attention heads by
    tensor-parallel rank, experts by expert-parallel rank)."""
    device = torch.device(device)
    # small models draw on the CPU (identical weights on every device, used by the CPU-vs-GPU tests); benchmark
    # shapes draw on the target device, where generating and quantising ~10^11 parameters takes seconds
    big = cfg.n_layers * cfg.n_experts * cfg.expert_ffn * cfg.d_model * 3 > 2e9 and device.type == "cuda"
    gen = torch.Generator(device=device if big else "cpu")
    gen.manual_seed(seed)
    cpu_fp32 = cfg.weight_format == "fp32"
    dt = torch.float32 if cpu_fp32 else torch.bfloat16
    d, hd, E, F = cfg.d_model, cfg.head_dim, cfg.n_experts, cfg.expert_ffn
    per = E // ep_size
    e_lo, e_hi = ep_rank * per, (ep_rank + 1) * per
    qs = cfg.q_size // tp_size
    if tp_size <= cfg.n_kv_heads:
        ks = cfg.kv_size // tp_size
        kv_lo, kv_hi = tp_rank * ks, (tp_rank + 1) * ks
    else:
        head = tp_rank * cfg.n_kv_heads // tp_size
        kv_lo, kv_hi = head * hd, (head + 1) * hd

    def rnd(shape):
        return (torch.randn(shape, generator=gen, dtype=torch.float32, device=device if big else "cpu") * std)

    quant = W4Weight.quantize_device if big else (lambda f, w: W4Weight.quantize(f, w, device, keep_file=False))

    embed = rnd((cfg.vocab, d)).to(dt).to(device)
    layers = []
    for _ in range(cfg.n_layers):
        wq, wk, wv, wo = rnd((cfg.q_size, d)), rnd((cfg.kv_size, d)), rnd((cfg.kv_size, d)), rnd((d, cfg.q_size))
        router = rnd((E, d))
        sinks = rnd((cfg.n_heads,)) * 10 if cfg.attention_sinks else None
        qkv = torch.cat([wq[tp_rank * qs:(tp_rank + 1) * qs], wk[kv_lo:kv_hi], wv[kv_lo:kv_hi]], dim=0)
        # expert weights are drawn one expert at a time so that a rank can skip (but still advance past) the others
        gu_local, dn_local = [], []
        for e in range(E):
            gu, dn = rnd((2 * F, d)), rnd((d, F))
            if e_lo <= e < e_hi:
                gu_local.append(gu)
                dn_local.append(dn)
        shared = {}
        if cfg.shared_expert_ffn > 0:
            fs = cfg.shared_expert_ffn
            sgu, sdn, sg = rnd((2 * fs, d)), rnd((d, fs)), rnd((1, d))
            router = torch.cat([router, sg, torch.zeros((7, d), dtype=router.dtype, device=router.device)], dim=0)
            shared = dict(shared_gate_up=LinearWeight("dense", sgu.to(dt).contiguous().to(device)),
                          shared_down=LinearWeight("dense", sdn.to(dt).contiguous().to(device)))
        layers.append(MoeLayerWeights(**shared, 
            attn_norm=torch.ones(d, dtype=dt, device=device),
            qkv=LinearWeight("dense", qkv.to(dt).contiguous().to(device)),
            o=LinearWeight("dense", wo[:, tp_rank * qs:(tp_rank + 1) * qs].to(dt).contiguous().to(device)),
            sinks=None if sinks is None else sinks[tp_rank * (cfg.n_heads // tp_size):(tp_rank + 1) * (cfg.n_heads // tp_size)]
            .float().contiguous().to(device),
            mlp_norm=torch.ones(d, dtype=dt, device=device),
            router=LinearWeight("dense", router.to(dt).contiguous().to(device)),
            gate_up=quant(cfg.expert_format, torch.stack(gu_local)),
            down=quant(cfg.expert_format, torch.stack(dn_local))))
        del gu_local, dn_local
    final_norm = torch.ones(d, dtype=dt, device=device)
    head = rnd((cfg.vocab, d))
    vo = 0
    if tp_size > 1:
        vs = (cfg.vocab + tp_size - 1) // tp_size
        vo = tp_rank * vs
        head = head[vo:min(cfg.vocab, vo + vs)]
    return MoeWeights(embed, layers, final_norm, LinearWeight("dense", head.to(dt).contiguous().to(device)), vo)


class MoeModel:
    def __init__(self, cfg: ModelConfig, weights: MoeWeights, tp=None, ep=None):
        self.cfg, self.w = cfg, weights
        self.tp = tp or NoTP()
        self.ep = ep or NoEP()
        t = self.tp.size
        self.hq = cfg.n_heads // t
        self.hkv = max(1, cfg.n_kv_heads // t)
        self.e_lo, self.e_hi = self.ep.expert_range(cfg.n_experts)

    @property
    def local_kv_heads(self) -> int:
        return self.hkv

    def hidden(self, b: ForwardBatch, cache) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        hd = cfg.head_dim
        h = ops.embedding(w.embed, b.tokens, cfg.embedding_scale)
        for li, lw in enumerate(w.layers):
            kv = cache.layer(li)
            x = ops.rmsnorm(h, lw.attn_norm, cfg.rms_eps, cfg.norm_offset_one)
            qkv = ops.linear(x, lw.qkv)
            q = ops.rope_kv_append(qkv, b.positions, b.seq_index, b.block_table, kv, self.hq, self.hkv, hd, cfg.rope_theta,
                                   cfg.rotary_dim)
            a = ops.attention(q, kv, b, self.hq, self.hkv, hd, window=cfg.layer_window(li), qkv=qkv, sinks=lw.sinks)
            h = self.tp.row_linear(a, lw.o, h)
            x = ops.rmsnorm(h, lw.mlp_norm, cfg.rms_eps, cfg.norm_offset_one)
            logits = ops.linear(x, lw.router)
            idx, rw = M.route(logits[:, :cfg.n_experts], cfg.top_k)
            h = self.ep.experts_combine(x, idx, rw, lw.gate_up, lw.down, cfg.act, self.e_lo, self.e_hi, h)
            if lw.shared_gate_up is not None:
                # replicated on every rank: the shared expert is a few percent of a layer's bytes
                sh = ops.linear(ops.gated_act(ops.linear(x, lw.shared_gate_up), cfg.act), lw.shared_down)
                h = M.shared_add(h, sh, logits[:, cfg.n_experts])
        return h

    def _keep(self, h: torch.Tensor) -> torch.Tensor:
        """Remembers the residual stream of the last forward (all rows, before the final norm) for consumers such
        as a multi-token-prediction head; a reference, not a copy."""
        self.last_hidden = h
        return h

    def logits(self, h: torch.Tensor, b: ForwardBatch) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        if b.logit_rows is not None:
            h = h.index_select(0, b.logit_rows)
        x = ops.rmsnorm(h, w.final_norm, cfg.rms_eps, cfg.norm_offset_one)
        return ops.linear(x, w.lm_head)

    def forward(self, b: ForwardBatch, cache) -> torch.Tensor:
        return self.tp.gather_logits(self.logits(self._keep(self.hidden(b, cache)), b))

    def greedy(self, b: ForwardBatch, cache) -> torch.Tensor:
        return self.tp.argmax(self.logits(self._keep(self.hidden(b, cache)), b), self.w.vocab_offset)


def qwen35_moe_shape(layers: int = 40) -> ModelConfig:
    """Qwen3.5-MoE-class layer geometry as the reference's expert kernels fix it (hidden 2048, 256 experts top-8,
    expert and shared-expert width 512: native/hip/src/moe_expert_kernel_internal.hpp:10-13), with plain GQA
    attention in every layer."""
    return ModelConfig(name="qwen35-moe", family="moe", n_layers=layers, d_model=2048, n_heads=16, n_kv_heads=2, head_dim=128,
                       ffn=512, vocab=151936, rope_theta=1e7, rms_eps=1e-6, weight_format="bf16", kv_format="bf16",
                       n_experts=256, top_k=8, expert_ffn=512, shared_expert_ffn=512, expert_format="mxfp4",
                       max_context=8192)


def tiny_shared_moe() -> ModelConfig:
    """CPU-checkable Qwen3.5-MoE-style layer: 256 experts top-8 plus the gated shared expert, small widths."""
    return ModelConfig(name="tiny-shared-moe", family="moe", n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64,
                       ffn=128, vocab=1024, weight_format="bf16", kv_format="bf16", n_experts=256, top_k=8, expert_ffn=128,
                       shared_expert_ffn=128, expert_format="mxfp4", max_context=256)


def tiny_moe() -> ModelConfig:
    """CPU-checkable MoE: 2 layers, 8 experts top-2, windowed + full attention with sinks."""
    return ModelConfig(name="tiny-moe", family="moe", n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256,
                       vocab=1024, weight_format="bf16", kv_format="bf16", sliding_window=16, window_layers=[True, False],
                       attention_sinks=True, n_experts=8, top_k=2, expert_ffn=256, expert_format="mxfp4", max_context=256)

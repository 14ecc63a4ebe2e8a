"""Qwen3.5-class hybrid decoder: gated-delta-net (linear attention) layers with every N-th layer full attention.

Full-attention layer: RMSNorm(1 + w) -> q | k | v (+ gate) projections -> per-head q/k RMSNorm(1 + w) -> rotary on
the first `rotary_dim` channels -> paged causal attention -> sigmoid(gate) * attention -> o projection.
GDN layer: RMSNorm -> in-projection to (q | k | v), z, b, a -> causal depthwise conv + SiLU on q|k|v with a rolling
state -> gated delta-rule recurrence fused with the output RMSNorm and SiLU(z) -> out projection.  Both are
followed by a SwiGLU MLP.  (Reference layer recipe: crates/sllm-core/src/qwen_graph.rs
`linear.{qkv,z,b,a}_matmul -> linear_attention_state -> linear.out_matmul`; kernels K16, K27, K28.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..engine.batch import ForwardBatch
from ..ops import gdn as G
from ..ops.core import LinearWeight
from .config import ModelConfig
from .llama import NoTP


@dataclass
class Qwen35Layer:
    kind: str                       # full | gdn
    in_norm: torch.Tensor
    mlp_norm: torch.Tensor
    gate_up: Optional[LinearWeight] = None
    down: Optional[LinearWeight] = None
    # full attention
    qkv: Optional[LinearWeight] = None
    gate: Optional[LinearWeight] = None
    o: Optional[LinearWeight] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    # gated delta net
    in_proj: Optional[LinearWeight] = None      # -> [qkv width | z (v_heads * hd) | b (v_heads) | a (v_heads)] (padded to 8)
    conv_w: Optional[torch.Tensor] = None       # [qkv width, taps]
    a_log: Optional[torch.Tensor] = None        # fp32 [v_heads]
    dt_bias: Optional[torch.Tensor] = None      # bf16 [v_heads]
    out_norm: Optional[torch.Tensor] = None     # fp32 [hd]
    out_proj: Optional[LinearWeight] = None
    # sparse MLP (Qwen3.5-MoE): replaces gate_up / down when the configuration has experts.  `router` holds the
    # expert rows, then the shared-expert gate vector, then zero padding to a multiple of 8
    router: Optional[LinearWeight] = None
    exp_gate_up: Optional[object] = None        # W4Weight, local experts, [2 * expert_ffn, d] each
    exp_down: Optional[object] = None           # W4Weight, local experts, [d, expert_ffn] each
    shared_gate_up: Optional[LinearWeight] = None
    shared_down: Optional[LinearWeight] = None


@dataclass
class Qwen35Weights:
    embed: torch.Tensor
    layers: list
    final_norm: torch.Tensor
    lm_head: LinearWeight
    vocab_offset: int = 0


def _head_rows(w: torch.Tensor, segments: list, tp_size: int, tp_rank: int) -> torch.Tensor:
    """Row shard of a weight whose rows are consecutive segments of (heads, rows per head): every segment gives the
    rank its contiguous share of heads."""
    if tp_size == 1:
        return w
    out, r0 = [], 0
    for heads, per in segments:
        if heads % tp_size:
            raise ValueError(f"{heads} heads do not divide over {tp_size} tensor-parallel ranks")
        loc = heads // tp_size
        out.append(w[r0 + tp_rank * loc * per:r0 + (tp_rank + 1) * loc * per])
        r0 += heads * per
    return torch.cat(out, dim=0)


def init_random_qwen35_weights(cfg: ModelConfig, device, seed: int = 0, std: float = 0.02, tp_size: int = 1,
                               tp_rank: int = 0, ep_size: int = 1, ep_rank: int = 0) -> Qwen35Weights:
    """Every rank draws the full tensors from the same generator and keeps its shard: attention and gated-delta-net
    layers are sharded by head, the dense MLP by intermediate channel, routed experts by expert range; norms,
    embedding, output matrix, router and shared expert are replicated."""
    device = torch.device(device)
    # benchmark shapes with routed experts (~10^10 parameters) draw and quantise on the target device; everything
    # else draws on the CPU so that every device sees identical weights
    big = cfg.n_layers * cfg.n_experts * cfg.expert_ffn * cfg.d_model * 3 > 2e9 and device.type == "cuda"
    gen = torch.Generator(device=device if big else "cpu")
    gen.manual_seed(seed)
    dt = torch.float32 if cfg.weight_format == "fp32" else torch.bfloat16
    d, hd = cfg.d_model, cfg.head_dim
    ghd, vh, qh = cfg.gdn_head_dim, cfg.gdn_heads, cfg.gdn_qk_heads
    width = (2 * qh + vh) * ghd

    def rnd(shape, s=std):
        return (torch.randn(shape, generator=gen, dtype=torch.float32, device=device if big else "cpu") * s)

    fp8 = cfg.weight_format == "fp8"

    def lin(w):
        """Projection matrices: bf16, or block-scaled FP8 (E4M3 + one fp32 scale per 1 x 128 block) when the
        configuration asks for FP8 weights; norms, convolution taps, gates' bias vectors and the router stay bf16."""
        w = w.to(dt).contiguous().to(device)
        if fp8:
            if w.is_cuda:
                q = ops.quant_fp8(w)
                return LinearWeight("fp8", q.data, q.scale)
            return LinearWeight.from_dense(w.float(), "fp8")
        return LinearWeight("dense", w)

    def lin_bf16(w):
        return LinearWeight("dense", w.to(dt).contiguous().to(device))

    def vec(v, dtype=None):
        return v.to(dtype or dt).contiguous().to(device)

    def rows(w, segments):
        return _head_rows(w, segments, tp_size, tp_rank)

    def cols(w, segments):
        return _head_rows(w.t(), segments, tp_size, tp_rank).t()

    f = cfg.ffn
    E = cfg.n_experts
    if E % ep_size:
        raise ValueError(f"{E} experts do not divide over {ep_size} expert-parallel ranks")
    e_lo, e_hi = ep_rank * (E // ep_size), (ep_rank + 1) * (E // ep_size)

    def sparse_mlp():
        from ..ops.w4 import W4Weight
        F, fs = cfg.expert_ffn, cfg.shared_expert_ffn
        router = rnd((E, d))
        gu_local, dn_local = [], []
        for e in range(E):                       # every rank advances the generator past every expert
            gu, dn = rnd((2 * F, d)), rnd((d, F))
            if e_lo <= e < e_hi:
                gu_local.append(gu)
                dn_local.append(dn)
        out = {}
        if fs > 0:
            sgu, sdn, sg = rnd((2 * fs, d)), rnd((d, fs)), rnd((1, d))
            router = torch.cat([router, sg, torch.zeros((7, d), device=router.device)], dim=0)
            out.update(shared_gate_up=lin(sgu), shared_down=lin(sdn))
        quant = W4Weight.quantize_device if big else (lambda f, w: W4Weight.quantize(f, w, device, keep_file=False))
        out.update(router=lin_bf16(router), exp_gate_up=quant(cfg.expert_format, torch.stack(gu_local)),
                   exp_down=quant(cfg.expert_format, torch.stack(dn_local)))
        return out

    layers = []
    for i in range(cfg.n_layers):
        common = dict(in_norm=vec(rnd((d,), 0.05)), mlp_norm=vec(rnd((d,), 0.05)))
        if E > 0:
            common.update(sparse_mlp())
        else:
            common.update(gate_up=lin(rows(rnd((2 * f, d)), [(f, 1), (f, 1)])), down=lin(cols(rnd((d, f)), [(f, 1)])))
        if (i + 1) % cfg.full_attention_interval == 0:
            hq, hkv = cfg.n_heads, cfg.n_kv_heads
            qkv = rows(rnd((cfg.q_size + 2 * cfg.kv_size, d)), [(hq, hd), (hkv, hd), (hkv, hd)])
            gate = rows(rnd((cfg.q_size, d)), [(hq, hd)]) if cfg.attn_output_gate else None
            layers.append(Qwen35Layer("full", qkv=lin(qkv), gate=lin(gate) if gate is not None else None,
                                      o=lin(cols(rnd((d, cfg.q_size)), [(hq, hd)])),
                                      q_norm=vec(rnd((hd,), 0.05), torch.bfloat16 if dt != torch.float32 else dt),
                                      k_norm=vec(rnd((hd,), 0.05), torch.bfloat16 if dt != torch.float32 else dt), **common))
        else:
            n_in = width + vh * ghd + 2 * vh
            segs = [(qh, ghd), (qh, ghd), (vh, ghd), (vh, ghd), (vh, 1), (vh, 1)]
            w_loc = rows(rnd((n_in, d)), segs)
            w_in = torch.zeros(((w_loc.shape[0] + 7) // 8 * 8, d), device=w_loc.device)
            w_in[:w_loc.shape[0]] = w_loc
            conv = rows(rnd((width, cfg.gdn_conv_kernel), 0.3), segs[:3])
            layers.append(Qwen35Layer("gdn", in_proj=lin(w_in), conv_w=vec(conv),
                                      a_log=vec(rows(rnd((vh,), 0.5), [(vh, 1)]), torch.float32),
                                      dt_bias=vec(rows(rnd((vh,), 0.5), [(vh, 1)])),
                                      out_norm=vec(1.0 + rnd((ghd,), 0.05), torch.float32),
                                      out_proj=lin(cols(rnd((d, vh * ghd)), [(vh, ghd)])), **common))
    embed = rnd((cfg.vocab, d)).to(dt).to(device)
    head = embed if cfg.tie_embeddings else rnd((cfg.vocab, d)).to(dt).contiguous().to(device)
    head_w = LinearWeight("dense", head)
    if fp8 and not cfg.tie_embeddings:
        head_w = lin(head)
    return Qwen35Weights(embed, layers, vec(rnd((d,), 0.05)), head_w, 0)


class Qwen35Model:
    def __init__(self, cfg: ModelConfig, weights: Qwen35Weights, tp=None, ep=None):
        from ..parallel.ep import NoEP
        self.cfg, self.w = cfg, weights
        self.tp = tp or NoTP()
        self.ep = ep or NoEP()
        self.e_lo, self.e_hi = self.ep.expert_range(cfg.n_experts) if cfg.n_experts else (0, 0)
        n = self.tp.size
        for name, v in (("n_heads", cfg.n_heads), ("n_kv_heads", cfg.n_kv_heads), ("gdn_heads", cfg.gdn_heads),
                        ("gdn_qk_heads", cfg.gdn_qk_heads), ("ffn", cfg.ffn if not cfg.n_experts else n)):
            if v % n:
                raise ValueError(f"{name} = {v} does not divide over {n} tensor-parallel ranks")
        # heads of this rank (attention and gated-delta-net layers are sharded by head)
        self.hq, self.hkv = cfg.n_heads // n, cfg.n_kv_heads // n
        self.vh, self.qh = cfg.gdn_heads // n, cfg.gdn_qk_heads // n

    @property
    def local_kv_heads(self) -> int:
        return self.hkv

    def _mlp(self, h, lw):
        cfg = self.cfg
        if lw.router is None:
            x = ops.rmsnorm(h, lw.mlp_norm, cfg.rms_eps, cfg.norm_offset_one, quant=lw.gate_up.kind == "fp8")
            act = ops.gated_act(ops.linear(x, lw.gate_up), cfg.act, quant=lw.down.kind == "fp8")
            return self.tp.row_linear(act, lw.down, h)
        x = ops.rmsnorm(h, lw.mlp_norm, cfg.rms_eps, cfg.norm_offset_one)
        # routed experts (softmax over the selected logits = softmax over all, renormalised over the selection) plus
        # the always-on shared expert under its sigmoid gate (crates/sllm-core/src/qwen35_moe.rs:1576-1600)
        from ..ops import moe as M
        logits = ops.linear(x, lw.router)
        idx, rw = M.route(logits[:, :cfg.n_experts], cfg.top_k)
        h = self.ep.experts_combine(x, idx, rw, lw.exp_gate_up, lw.exp_down, cfg.act, self.e_lo, self.e_hi, h)
        if lw.shared_gate_up is not None:
            sh = ops.linear(ops.gated_act(ops.linear(x, lw.shared_gate_up), cfg.act), lw.shared_down)
            h = M.shared_add(h, sh, logits[:, cfg.n_experts])
        return h

    def hidden(self, b: ForwardBatch, cache) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        hd, ghd, vh, qh = cfg.head_dim, cfg.gdn_head_dim, self.vh, self.qh
        width = (2 * qh + vh) * ghd
        if b.row_off is None or b.slots is None:
            raise ValueError("the hybrid family needs row offsets and state slots in the batch")
        h = ops.embedding(w.embed, b.tokens, cfg.embedding_scale)
        for li, lw in enumerate(w.layers):
            first = lw.qkv if lw.kind == "full" else lw.in_proj
            # FP8 projections take the normalised row as E4M3 + block scales, written by the norm kernel itself
            x = ops.rmsnorm(h, lw.in_norm, cfg.rms_eps, cfg.norm_offset_one, quant=first.kind == "fp8")
            if lw.kind == "full":
                kv = cache.layer(li)
                qkv = ops.linear(x, lw.qkv)
                qkv = G.qk_headnorm(qkv, self.hq, self.hkv, hd, lw.q_norm, lw.k_norm, cfg.rms_eps, True)
                q = ops.rope_kv_append(qkv, b.positions, b.seq_index, b.block_table, kv, self.hq, self.hkv, hd, cfg.rope_theta,
                                       cfg.rotary_dim)
                a = ops.paged_attention(q, kv, b.block_table, b.seq_index, b.kv_lens, self.hq, self.hkv, hd, max_kv=b.max_kv)
                if lw.gate is not None:
                    a = ops.elementwise("sigmoid_mul", a.contiguous(), ops.linear(x, lw.gate))
                h = self.tp.row_linear(a, lw.o, h)
            else:
                conv_state, rec_state = cache.gdn(li)
                p = ops.linear(x, lw.in_proj)
                # column slices of the projection output: the kernels take the row stride (no copies)
                qkv = p[:, :width]
                z = p[:, width:width + vh * ghd]
                bb = p[:, width + vh * ghd:width + vh * ghd + vh]
                aa = p[:, width + vh * ghd + vh:width + vh * ghd + 2 * vh]
                qkv = G.conv_silu(qkv, lw.conv_w, conv_state, b.row_off, b.slots)
                o = G.recurrent(qkv, z, bb, aa, lw.a_log, lw.dt_bias, lw.out_norm, rec_state, b.row_off, b.slots, qh, vh, ghd)
                h = self.tp.row_linear(o, lw.out_proj, h)
            h = self._mlp(h, lw)
        return h

    def _keep(self, h: torch.Tensor) -> torch.Tensor:
        """Remembers the residual stream of the last forward (all rows, before the final norm) for consumers such
        as a multi-token-prediction head; a reference, not a copy."""
        self.last_hidden = h
        return h

    def logits(self, h, b):
        cfg, w = self.cfg, self.w
        if b.logit_rows is not None:
            h = h.index_select(0, b.logit_rows)
        x = ops.rmsnorm(h, w.final_norm, cfg.rms_eps, cfg.norm_offset_one)
        return ops.linear(x, w.lm_head)

    def forward(self, b, cache):
        return self.logits(self._keep(self.hidden(b, cache)), b)

    def greedy(self, b, cache):
        return ops.argmax(self.logits(self._keep(self.hidden(b, cache)), b))


def qwen35_moe_hybrid_shape(layers: int = 40) -> ModelConfig:
    """Qwen3.5-MoE as the reference pins it (crates/sllm-core/src/qwen35_moe.rs:1177-1189): 40 layers of width 2048,
    every fourth one full attention (16 heads, 2 kv heads, 256 wide), the others gated delta nets; every MLP is 256
    MXFP4 experts of width 512 with 8 selected per token plus a gated shared expert of width 512; vocabulary 248 320."""
    return ModelConfig(name="qwen35-moe-hybrid", family="qwen35", n_layers=layers, d_model=2048, n_heads=16, n_kv_heads=2,
                       head_dim=256, ffn=512, vocab=248320, rope_theta=1e7, rotary_dim=64, rms_eps=1e-6, norm_offset_one=True,
                       weight_format="bf16", kv_format="bf16", qk_norm=True, full_attention_interval=4, gdn_heads=32,
                       gdn_qk_heads=16, gdn_head_dim=128, gdn_conv_kernel=4, attn_output_gate=True, n_experts=256, top_k=8,
                       expert_ffn=512, shared_expert_ffn=512, expert_format="mxfp4", max_context=8192)


def tiny_qwen35_moe() -> ModelConfig:
    """CPU-checkable hybrid with a sparse MLP: the tiny hybrid's layers, 8 experts of width 128 with 2 selected, and
    the gated shared expert."""
    c = tiny_qwen35()
    c.name, c.n_experts, c.top_k, c.expert_ffn, c.shared_expert_ffn, c.expert_format = "tiny-qwen35-moe", 8, 2, 128, 128, "mxfp4"
    c.d_model = 128
    return c


def tiny_qwen35() -> ModelConfig:
    """CPU-checkable hybrid: 4 layers (3 GDN + 1 full), 1 GDN q/k head and 2 value heads of 128."""
    return ModelConfig(name="tiny-qwen35", family="qwen35", n_layers=4, d_model=128, n_heads=2, n_kv_heads=1, head_dim=64, ffn=256,
                       vocab=512, rope_theta=1e7, rotary_dim=32, rms_eps=1e-6, norm_offset_one=True, weight_format="bf16",
                       kv_format="bf16", qk_norm=True, full_attention_interval=4, gdn_heads=2, gdn_qk_heads=1, gdn_head_dim=128,
                       gdn_conv_kernel=4, attn_output_gate=True, max_context=128)

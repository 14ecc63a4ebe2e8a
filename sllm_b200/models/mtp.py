"""Multi-token-prediction (MTP) head: one extra decoder layer that drafts the token after next from the target's
own hidden state, sharing the target's embedding and output matrices.

Position i of the head takes the pair (embedding of token i+1, target hidden row i): both are RMS-normalised,
concatenated and projected back to d_model (`fc`, [d, 2d]); the result passes one full decoder layer (its own KV
cache, one layer deep) and the head's final norm, and the shared output matrix turns it into logits for token
i+2.  Further drafts feed the head its own output row in place of the target's.  The component mirrors the
reference's 15-tensor `mtp.*` manifest (fc, pre_fc_norm_embedding, pre_fc_norm_hidden, one layer, norm;
crates/sllm-core/src/qwen_mtp.rs:184-202) and its executor (propose on the target's last hidden state, verify
with the target, rewind and replay accepted inputs; crates/sllm-core/src/generation.rs:1305-1516).  Exactness
does not depend on the head: the target's verify rows are the only source of visible tokens.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..cache.paged import PagedKVCache
from ..ops.core import LinearWeight
from .config import ModelConfig
from .llama import LlamaModel, LlamaWeights, init_random_weights

MAX_MTP_WIDTH = 8


@dataclass
class MtpWeights:
    fc: LinearWeight                 # [d, 2d]: (normalised embedding | normalised hidden) -> d
    norm_embedding: torch.Tensor     # [d]
    norm_hidden: torch.Tensor        # [d]
    layer: object                    # models.llama.LayerWeights of the head's decoder layer
    norm: torch.Tensor               # [d] final norm of the head


def mtp_layer_config(cfg: ModelConfig) -> ModelConfig:
    """The head's one-layer decoder: the target's attention / MLP shape, full attention, dense weights."""
    c = copy.deepcopy(cfg)
    c.name = cfg.name + "-mtp"
    c.family = "llama"
    c.n_layers = 1
    c.sliding_window, c.window_layers = 0, None
    c.n_experts = c.top_k = 0
    c.full_attention_interval = 0
    if c.weight_format not in ("fp32", "bf16"):
        c.weight_format = "bf16"
    return c


def init_random_mtp_weights(cfg: ModelConfig, device, seed: int = 1) -> MtpWeights:
    device = torch.device(device)
    lc = mtp_layer_config(cfg)
    base = init_random_weights(lc, device, seed)
    dt = torch.float32 if lc.weight_format == "fp32" else torch.bfloat16
    gen = torch.Generator().manual_seed(seed + 7919)
    d = cfg.d_model
    fc = (torch.randn((d, 2 * d), generator=gen) * (0.5 / d ** 0.5)).to(dt).to(device)
    ne = (1.0 + 0.05 * torch.randn((d,), generator=gen)).to(dt).to(device)
    nh = (1.0 + 0.05 * torch.randn((d,), generator=gen)).to(dt).to(device)
    if cfg.norm_offset_one:
        ne, nh = ne - 1.0, nh - 1.0
    return MtpWeights(LinearWeight("dense", fc.contiguous()), ne, nh, base.layers[0], base.final_norm)


class MtpHead:
    """The head on its own one-layer engine; `embeds` builds its inputs, the engine keeps its KV per sequence."""

    def __init__(self, target_engine, weights: MtpWeights, max_batch: Optional[int] = None):
        from ..engine.engine import Engine
        tm = target_engine.model
        if getattr(getattr(tm, "tp", None), "size", 1) != 1:
            raise ValueError("the MTP head runs without tensor parallelism")
        self.target = target_engine
        self.cfg = mtp_layer_config(target_engine.cfg)
        self.w = weights
        tw = tm.w
        inner_w = LlamaWeights(tw.embed, [weights.layer], weights.norm, tw.lm_head, getattr(tw, "vocab_offset", 0))
        model = LlamaModel(self.cfg, inner_w, None)
        # the shared output matrix may be FP8 while the head's own layer is dense: quantise only the logits input
        model.quant = False
        self._head_quant = getattr(tw.lm_head, "kind", "dense") == "fp8"
        if self._head_quant:
            cfg = self.cfg

            def logits(h, b, _m=model):
                if b.logit_rows is not None:
                    h = h.index_select(0, b.logit_rows)
                x = ops.rmsnorm(h, _m.w.final_norm, cfg.rms_eps, cfg.norm_offset_one, quant=True)
                return ops.linear(x, _m.w.lm_head)
            model.logits = logits
        mb = max_batch or target_engine.max_batch
        pages = mb * ((self.cfg.max_context + self.cfg.page_size - 1) // self.cfg.page_size) + 8
        cache = PagedKVCache(self.cfg, pages, target_engine.device, kv_heads=model.local_kv_heads)
        self.engine = Engine(self.cfg, model, cache, target_engine.device, max_batch=mb, use_cuda_graphs=False)

    def embeds(self, tokens: torch.Tensor, hidden: torch.Tensor) -> torch.Tensor:
        """fc(cat(norm(embedding(tokens)), norm(hidden))) for rows of (next token, hidden) pairs."""
        cfg, w = self.target.cfg, self.w
        e = ops.embedding(self.target.model.w.embed, tokens, cfg.embedding_scale)
        xe = ops.rmsnorm(e, w.norm_embedding, cfg.rms_eps, cfg.norm_offset_one)
        xh = ops.rmsnorm(hidden.to(e.dtype), w.norm_hidden, cfg.rms_eps, cfg.norm_offset_one)
        return ops.linear(torch.cat([xe, xh], dim=-1).contiguous(), w.fc)


class MtpDraftProvider:
    """Draft provider for `SpeculativeDecoder`: greedy drafts from an `MtpHead`.

    Per target sequence the head keeps a sequence of its own whose position i holds the pair (token i+1, target
    hidden i).  A round first catches up on the positions the target has computed since the last round (with the
    target's logged hidden rows), then drafts recurrently, then forgets the recurrent rows again: they were
    computed from the head's own hidden rows and are replaced by the target's after verification."""

    def __init__(self, head: MtpHead, width: int = 2):
        if not 1 <= width <= MAX_MTP_WIDTH:
            raise ValueError("draft width must be in 1..8")
        self.head, self.width = head, width
        head.target.keep_hidden = True
        self.identity = f"mtp:{head.cfg.name}:{width}"
        self._seqs: dict = {}

    def propose_seqs(self, seqs: list, width: Optional[int] = None) -> list:
        w = min(width or self.width, self.width)
        head, eng, tgt = self.head, self.head.engine, self.head.target
        dev = tgt.device
        inner, tok_rows, hid_rows = [], [], []
        for s in seqs:
            n = s.num_computed                      # target positions 0..n-1 are computed; token n is the newest
            if n < 1 or len(s.tokens) != n + 1:
                raise ValueError("MTP drafting needs exactly one uncomputed token per sequence")
            ent = self._seqs.get(id(s))
            if ent is None:
                # the head starts at the first position whose hidden row the target logged: 0 normally, later when
                # the request forked a cached prefix (the head then sees a shorter history; rotary attention only
                # depends on position differences, so its rows stay consistent with one another)
                first = tgt.hidden_start(s)
                if first is None or first >= n:
                    raise ValueError("the target engine logged no hidden rows for this sequence")
                ent = self._seqs[id(s)] = [eng.new_sequence([]), first]
            m, off = ent
            c = min(m.num_computed, n - off)
            if m.tokens[:c] != s.tokens[off + 1:off + c + 1]:
                # the target's history changed under us (a context shift): restart from the rows still logged
                first = tgt.hidden_start(s)
                if first is None or first >= n:
                    raise ValueError("the target engine logged no hidden rows for this sequence")
                ent[1] = off = first
                c = 0
            eng.rollback(m, c)
            m.tokens = list(s.tokens[off + 1:n + 1])
            m.prompt = list(m.tokens)
            tok_rows.extend(s.tokens[off + c + 1:n + 1])
            hid_rows.append(tgt.take_hidden(s, off + c, n))
            inner.append(m)
        toks = torch.tensor(tok_rows, dtype=torch.int32, device=dev)
        hid = torch.cat(hid_rows, 0) if len(hid_rows) > 1 else hid_rows[0]
        rows = eng.extend(inner, embeds=head.embeds(toks, hid))
        drafts = [[r[-1]] for r in rows]
        # row offsets of each sequence's last row in the flattened batch
        ends, r0 = [], 0
        for r in rows:
            r0 += len(r)
            ends.append(r0 - 1)
        last = eng.model.last_hidden.index_select(0, torch.tensor(ends, device=dev))
        for _ in range(w - 1):
            for m, d in zip(inner, drafts):
                m.tokens.append(d[-1])
            nxt = torch.tensor([d[-1] for d in drafts], dtype=torch.int32, device=dev)
            rows = eng.extend(inner, embeds=head.embeds(nxt, last))
            last = eng.model.last_hidden
            for d, r in zip(drafts, rows):
                d.append(r[-1])
        for s, m in zip(seqs, inner):
            # keep only rows computed from the target's hidden states
            eng.rollback(m, s.num_computed - self._seqs[id(s)][1])
        return drafts

    def propose(self, tokens: list, width: Optional[int] = None) -> list:
        raise NotImplementedError("the MTP head drafts from engine sequences (propose_seqs)")

    def release(self, key) -> None:
        ent = self._seqs.pop(key, None)
        if ent is not None:
            self.head.engine.free_sequence(ent[0])

"""Llama-style decoder in plain PyTorch: bf16 weights and activations, contiguous bf16 KV cache,
`scaled_dot_product_attention`, tensor parallelism with `torch.distributed.all_reduce` after the row-parallel
projections.  Weights are drawn with the same generator sequence as the engine's random initialiser, so both
arms run the same network (this arm keeps the values in bf16 instead of FP8)."""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F


class TorchLlama:
    def __init__(self, cfg, device, seed: int = 0, tp_size: int = 1, tp_rank: int = 0, max_batch: int = 32, group=None):
        self.cfg, self.device, self.tp, self.rank, self.group = cfg, torch.device(device), tp_size, tp_rank, group
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        d, hd = cfg.d_model, cfg.head_dim
        self.hq, self.hkv = cfg.n_heads // tp_size, max(1, cfg.n_kv_heads // tp_size)

        def rnd(shape):
            return (torch.randn(shape, generator=gen, device=self.device, dtype=torch.float32) * 0.02).to(torch.bfloat16)

        def shard_rows(w, n):
            s = n // tp_size
            return w[tp_rank * s:(tp_rank + 1) * s]

        self.embed = rnd((cfg.vocab, d))
        self.layers = []
        for _ in range(cfg.n_layers):
            wq, wk, wv, wo = rnd((cfg.q_size, d)), rnd((cfg.kv_size, d)), rnd((cfg.kv_size, d)), rnd((d, cfg.q_size))
            wg, wu, wd = rnd((cfg.ffn, d)), rnd((cfg.ffn, d)), rnd((d, cfg.ffn))
            qs, fs = cfg.q_size // tp_size, cfg.ffn // tp_size
            if tp_size <= cfg.n_kv_heads:
                wk, wv = shard_rows(wk, cfg.kv_size), shard_rows(wv, cfg.kv_size)
            else:
                h = tp_rank * cfg.n_kv_heads // tp_size
                wk, wv = wk[h * hd:(h + 1) * hd], wv[h * hd:(h + 1) * hd]
            self.layers.append(dict(
                qkv=torch.cat([shard_rows(wq, cfg.q_size), wk, wv]).contiguous(),
                o=wo[:, tp_rank * qs:(tp_rank + 1) * qs].contiguous(),
                gu=torch.cat([shard_rows(wg, cfg.ffn), shard_rows(wu, cfg.ffn)]).contiguous(),
                down=wd[:, tp_rank * fs:(tp_rank + 1) * fs].contiguous(),
                n1=torch.ones(d, device=self.device, dtype=torch.bfloat16), n2=torch.ones(d, device=self.device, dtype=torch.bfloat16)))
        self.final_norm = torch.ones(d, device=self.device, dtype=torch.bfloat16)
        head = rnd((cfg.vocab, d))
        vs = (cfg.vocab + tp_size - 1) // tp_size
        self.vocab_offset = tp_rank * vs if tp_size > 1 else 0
        self.head = head[self.vocab_offset:self.vocab_offset + vs].contiguous() if tp_size > 1 else head
        self.k = [torch.zeros(max_batch, self.hkv, cfg.max_context, hd, device=self.device, dtype=torch.bfloat16)
                  for _ in range(cfg.n_layers)]
        self.v = [torch.zeros_like(k) for k in self.k]
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=self.device).float() / hd))
        t = torch.arange(cfg.max_context, device=self.device).float()
        fr = torch.outer(t, inv)
        self.cos, self.sin = fr.cos(), fr.sin()

    def _norm(self, x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.rms_eps)).to(torch.bfloat16) * w

    def _rope(self, x, pos):          # x [B, T, H, hd], pos [B, T]
        hd = x.shape[-1]
        c, s = self.cos[pos].unsqueeze(2), self.sin[pos].unsqueeze(2)
        x1, x2 = x[..., :hd // 2].float(), x[..., hd // 2:].float()
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(torch.bfloat16)

    def _allreduce(self, y):
        if self.tp > 1:
            dist.all_reduce(y, group=self.group)
        return y

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, start: int) -> torch.Tensor:
        """tokens [B, T] at positions start .. start + T - 1 (same for every row); returns greedy next tokens [B]."""
        cfg = self.cfg
        b, t = tokens.shape
        hd = cfg.head_dim
        pos = torch.arange(start, start + t, device=self.device).unsqueeze(0).expand(b, t)
        h = self.embed[tokens]
        for li, w in enumerate(self.layers):
            x = self._norm(h, w["n1"])
            qkv = x @ w["qkv"].t()
            q, k, v = qkv.split([self.hq * hd, self.hkv * hd, self.hkv * hd], dim=-1)
            q = self._rope(q.view(b, t, self.hq, hd), pos).transpose(1, 2)
            k = self._rope(k.view(b, t, self.hkv, hd), pos).transpose(1, 2)
            v = v.view(b, t, self.hkv, hd).transpose(1, 2)
            self.k[li][:b, :, start:start + t] = k
            self.v[li][:b, :, start:start + t] = v
            kk, vv = self.k[li][:b, :, :start + t], self.v[li][:b, :, :start + t]
            a = F.scaled_dot_product_attention(q, kk, vv, is_causal=(t > 1 and start == 0), enable_gqa=True)
            a = a.transpose(1, 2).reshape(b, t, self.hq * hd)
            h = h + self._allreduce(a @ w["o"].t())
            x = self._norm(h, w["n2"])
            g, u = (x @ w["gu"].t()).chunk(2, dim=-1)
            h = h + self._allreduce((F.silu(g.float()).to(torch.bfloat16) * u) @ w["down"].t())
        x = self._norm(h[:, -1], self.final_norm)
        logits = (x @ self.head.t()).float()
        val, idx = logits.max(dim=-1)
        idx = idx + self.vocab_offset
        if self.tp > 1:
            vals = [torch.empty_like(val) for _ in range(self.tp)]
            idxs = [torch.empty_like(idx) for _ in range(self.tp)]
            dist.all_gather(vals, val, group=self.group)
            dist.all_gather(idxs, idx, group=self.group)
            v_all, i_all = torch.stack(vals), torch.stack(idxs)
            idx = i_all.gather(0, v_all.argmax(0, keepdim=True)).squeeze(0)
        return idx

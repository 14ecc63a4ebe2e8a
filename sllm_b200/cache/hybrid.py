"""KV pages for the full-attention layers plus O(1) recurrent state for the gated-delta-net layers.

A sequence owns one state slot for its lifetime: per GDN layer a rolling convolution window
[taps - 1, qkv width] (bf16) and a recurrent matrix [value heads, 128, 128] (fp32) - the reference's
`[3, 8192]` + `[32, 128, 128]` per layer (crates/sllm-core/src/linear_attention.rs).  The state always
describes the end of the sequence's computed tokens, so a prefix can be shared only at exactly that point and a
rewind needs a snapshot (`snapshot` / `restore`, used by speculative rollback and context rebuilds).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..models.config import ModelConfig
from .paged import PagedKVCache


class HybridCache(PagedKVCache):
    def __init__(self, cfg: ModelConfig, num_pages: int, device, max_seqs: int, kv_heads: Optional[int] = None,
                 tp_size: int = 1):
        """``tp_size``: the gated-delta-net heads (and with them the conv and recurrent state) are split over that
        many tensor-parallel ranks; this cache holds one rank's share."""
        self.full_layers = [i for i in range(cfg.n_layers) if (i + 1) % cfg.full_attention_interval == 0]
        self.gdn_layers = [i for i in range(cfg.n_layers) if i not in self.full_layers]
        import dataclasses
        kv_cfg = dataclasses.replace(cfg, n_layers=max(1, len(self.full_layers)))
        super().__init__(kv_cfg, num_pages, device, kv_heads)
        self._kv_index = {l: j for j, l in enumerate(self.full_layers)}
        self._gdn_index = {l: j for j, l in enumerate(self.gdn_layers)}
        hd = cfg.gdn_head_dim
        self.width = (2 * cfg.gdn_qk_heads + cfg.gdn_heads) // tp_size * hd
        n = max(1, len(self.gdn_layers))
        self.max_seqs = max_seqs
        self.conv_state = torch.zeros((n, max_seqs, cfg.gdn_conv_kernel - 1, self.width), dtype=torch.bfloat16 if
                                      torch.device(device).type == "cuda" or cfg.weight_format != "fp32" else torch.float32,
                                      device=device)
        self.rec_state = torch.zeros((n, max_seqs, cfg.gdn_heads // tp_size, hd, hd), dtype=torch.float32, device=device)
        self._free = list(range(max_seqs - 1, -1, -1))
        self.slot_of: dict = {}

    def layer(self, i: int):
        j = self._kv_index.get(i)
        return None if j is None else self._layers[j]

    def gdn(self, i: int):
        j = self._gdn_index[i]
        return self.conv_state[j], self.rec_state[j]

    # ---------------------------------------------------------------- slots
    def alloc_slot(self, seq_id: int) -> int:
        if not self._free:
            raise RuntimeError("no free recurrent-state slot")
        s = self._free.pop()
        self.slot_of[seq_id] = s
        self.conv_state[:, s].zero_()
        self.rec_state[:, s].zero_()
        return s

    def free_slot(self, seq_id: int) -> None:
        s = self.slot_of.pop(seq_id, None)
        if s is not None:
            self._free.append(s)

    def copy_slot(self, src_seq: int, dst_seq: int) -> None:
        a, b = self.slot_of[src_seq], self.slot_of[dst_seq]
        self.conv_state[:, b].copy_(self.conv_state[:, a])
        self.rec_state[:, b].copy_(self.rec_state[:, a])

    def snapshot(self, seq_id: int):
        s = self.slot_of[seq_id]
        return self.conv_state[:, s].clone(), self.rec_state[:, s].clone()

    def restore(self, seq_id: int, snap) -> None:
        s = self.slot_of[seq_id]
        self.conv_state[:, s].copy_(snap[0])
        self.rec_state[:, s].copy_(snap[1])

    def bytes_per_token(self) -> int:
        return super().bytes_per_token()

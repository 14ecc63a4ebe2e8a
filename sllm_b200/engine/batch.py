"""The flat token batch every model forward consumes.

Per-row positions, sequence indices and key counts are part of the kernel ABI from the start, so
that requests at different positions share one launch (continuous batching) and a speculative
block is just several rows of one sequence.  The reference keeps these as per-request scalars,
which is why its batch planner was never connected (docs/plans/main-plan.md:894-904).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class ForwardBatch:
    tokens: torch.Tensor        # int32 [T]
    positions: torch.Tensor     # int32 [T] absolute position of each token
    seq_index: torch.Tensor     # int32 [T] row of block_table that owns the token
    kv_lens: torch.Tensor       # int32 [T] keys visible to the token (position + 1)
    block_table: torch.Tensor   # int32 [S, max_blocks]
    logit_rows: Optional[torch.Tensor] = None  # int64 rows that need logits (None = all rows)
    max_kv: int = 0             # host-side upper bound on kv_lens, for split heuristics
    # Fresh-prompt prefill metadata (tokens of each sequence contiguous, starting at position 0):
    cu_seqlens: Optional[torch.Tensor] = None  # int32 [S + 1]
    max_seqlen: int = 0
    embeds: Optional[torch.Tensor] = None      # optional [T, d] input embeddings replacing the gather
    rope_pos3: Optional[torch.Tensor] = None   # optional int32 [3, T] temporal / height / width rotary positions
    cu_seqlens_host: Optional[list] = None     # the same offsets as a Python list (tile scheduling)
    prefill_tiles: Optional[torch.Tensor] = None  # cached tile table of the tensor-core prefill kernel
    # Recurrent-state (gated delta net) layers: rows of sequence s are row_off[s] .. row_off[s + 1], its state lives in
    # slot slots[s] of the state cache.
    row_off: Optional[torch.Tensor] = None     # int32 [S + 1]
    slots: Optional[torch.Tensor] = None       # int32 [S]

    @property
    def num_tokens(self) -> int:
        return self.tokens.numel()


def make_prefill_batch(prompts: list, block_table: torch.Tensor, device, start_positions: Optional[list] = None,
                       last_only: bool = True) -> ForwardBatch:
    """prompts: list of token-id lists, one per row of block_table."""
    toks, pos, sidx = [], [], []
    cu = [0]
    rows = []
    fresh = True
    for i, p in enumerate(prompts):
        s0 = 0 if start_positions is None else start_positions[i]
        fresh = fresh and s0 == 0
        toks.extend(p)
        pos.extend(range(s0, s0 + len(p)))
        sidx.extend([i] * len(p))
        cu.append(cu[-1] + len(p))
        rows.append(cu[-1] - 1)
    t = lambda x, dt=torch.int32: torch.tensor(x, dtype=dt, device=device)
    positions = t(pos)
    return ForwardBatch(
        tokens=t(toks), positions=positions, seq_index=t(sidx), kv_lens=positions + 1,
        block_table=block_table, logit_rows=t(rows, torch.int64) if last_only else None,
        max_kv=max(pos) + 1 if pos else 0, cu_seqlens=t(cu) if fresh else None,
        max_seqlen=max(len(p) for p in prompts) if prompts else 0, cu_seqlens_host=cu if fresh else None,
        row_off=t(cu))

"""Model executor: owns the weights, the paged KV cache and the CUDA-graph-captured decode step.

The public calls are ``prefill`` / ``decode`` on lists of ``Sequence`` objects (used by the
continuous-batching scheduler) and ``generate`` (batch convenience, used by the CLI and benchmarks).
A step is transactional in the reference's sense (crates/sllm-core/src/prepared_execution.rs:25,
docs/architecture/runtime.md:145-149): page storage is reserved before launch, and a sequence's
published length moves only after the step's results have been read back; any exception leaves the
published state untouched and marks only the affected sequences as failed.

Decode steps run from CUDA graphs, one per padded batch size, over static input buffers (tokens,
positions, key counts, block table); the host copies each step's inputs from pinned memory and
reads the sampled tokens back, which is the only per-step host/device traffic
(reference: 2 small H2D + 1 tiny D2H per step, docs/plans/main-plan.md:1297-1300).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from .. import ops
from ..cache.paged import OutOfPages, PagedKVCache
from ..models.config import ModelConfig
from .batch import ForwardBatch, make_prefill_batch


@dataclass
class Sequence:
    prompt: list
    seq_id: int = -1           # handle in the page pool
    tokens: list = field(default_factory=list)  # prompt + generated
    num_computed: int = 0      # tokens whose KV is published
    failed: Optional[str] = None
    user: object = None
    rope_delta: int = 0        # rotary position of token i = i + rope_delta once a multimodal prompt compressed it

    def __post_init__(self):
        if not self.tokens:
            self.tokens = list(self.prompt)

    @property
    def num_generated(self) -> int:
        return len(self.tokens) - len(self.prompt)


class EngineQuarantined(RuntimeError):
    """The engine gave up on the device (a bounded device wait ran out): it computes nothing further."""


# Buffers of quarantined engines whose device work could not be proven complete: kept referenced for the life of the
# process so that their memory is never handed to anyone else (reference: the "unowned cleanup state" of
# native/hip/src/runtime_impl.hpp, where memory of a failed stream is parked instead of freed).
_PARKED: list = []


class Engine:
    GRAPH_BATCHES = (1, 2, 4, 8, 16, 32, 64, 128)

    def __init__(self, cfg: ModelConfig, model, cache: PagedKVCache, device, max_batch: int = 64,
                 use_cuda_graphs: bool = True, tp=None):
        self.cfg = cfg
        self.model = model
        self.cache = cache
        self.device = torch.device(device)
        self.is_cuda = self.device.type == "cuda"
        self.max_batch = max_batch
        self.max_blocks = (cfg.max_context + cfg.page_size - 1) // cfg.page_size
        self.use_graphs = use_cuda_graphs and self.is_cuda
        self.tp = tp
        self.has_state = hasattr(cache, "alloc_slot")     # recurrent-state (gated delta net) layers present
        self._graphs: dict = {}
        self._graph_launches: dict = {}
        pin = self.is_cuda
        # host staging (pinned) and device-side static inputs
        self.h_tokens = torch.zeros(max_batch, dtype=torch.int32, pin_memory=pin)
        self.h_positions = torch.zeros(max_batch, dtype=torch.int32, pin_memory=pin)
        self.h_table = torch.zeros((max_batch, self.max_blocks), dtype=torch.int32, pin_memory=pin)
        self.h_out = torch.zeros(max_batch, dtype=torch.int32, pin_memory=pin)
        self.d_tokens = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self.d_positions = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self.d_kv_lens = torch.ones(max_batch, dtype=torch.int32, device=self.device)
        self.d_seq_index = torch.arange(max_batch, dtype=torch.int32, device=self.device)
        self.d_table = torch.zeros((max_batch, self.max_blocks), dtype=torch.int32, device=self.device)
        self.d_out = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self.h_slots = torch.zeros(max_batch, dtype=torch.int32, pin_memory=pin)
        self.d_slots = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self.d_row_off = torch.arange(max_batch + 1, dtype=torch.int32, device=self.device)
        self.d_logits = None
        # text rows after a multimodal prompt: rotary position = index + per-sequence delta, on all three axes
        self.h_rope_delta = torch.zeros(max_batch, dtype=torch.int32, pin_memory=pin)
        self.d_rope_delta = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self.d_rope3 = torch.zeros(3 * max_batch, dtype=torch.int32, device=self.device)
        self._rope3_on = False
        self.np_tokens = self.h_tokens.numpy()
        self.np_positions = self.h_positions.numpy()
        self._steps = 0
        self._table_key = None
        self.kernel_launches = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        # with keep_hidden set, prefill / extend log the final residual-stream row of every computed position per
        # sequence (consumed by a multi-token-prediction head through take_hidden)
        self.keep_hidden = False
        self._hidden_log: dict = {}
        self.quarantine: Optional[dict] = None     # set once by _enter_quarantine; the engine then refuses all work
        self._mem_mark = torch.cuda.memory_allocated(self.device) if self.is_cuda else 0

    # ------------------------------------------------------------------ failure containment and accounting
    def _guard(self) -> None:
        if self.quarantine is not None:
            raise EngineQuarantined(f"engine is quarantined: {self.quarantine['reason']}")

    def _enter_quarantine(self, reason: str, device_status: int = 0) -> None:
        """Stops the engine for good.  Captured graphs are dropped; the device is given one synchronize to prove that
        nothing of this engine is still running: only then may `release` free its memory, otherwise the buffers are
        parked for the life of the process."""
        if self.quarantine is not None:
            return
        completed = True
        if self.is_cuda:
            try:
                torch.cuda.synchronize(self.device)
            except RuntimeError:
                completed = False
        self._graphs.clear()
        self.quarantine = {"reason": reason, "device_status": int(device_status), "work_completed": completed,
                           "steps": self._steps}

    def release(self) -> dict:
        """Drops the engine's device memory (KV pages, staging) when that is safe; returns what happened to it."""
        cache_bytes = self.cache.values.numel() * self.cache.values.element_size() if hasattr(self.cache, "values") else 0
        if self.quarantine is not None and not self.quarantine["work_completed"]:
            _PARKED.append((self.cache, self.model, self._graphs))
            return {"freed_bytes": 0, "parked_bytes": cache_bytes}
        self._graphs.clear()
        if hasattr(self.cache, "values"):
            self.cache.values = self.cache.values.new_empty(0)
            if getattr(self.cache, "scales", None) is not None:
                self.cache.scales = self.cache.scales.new_empty(0)
            self.cache._layers = []
        if self.quarantine is None:
            self.quarantine = {"reason": "released", "device_status": 0, "work_completed": True, "steps": self._steps}
        return {"freed_bytes": cache_bytes, "parked_bytes": 0}

    def accounting(self) -> dict:
        """Bytes by category, and the allocator's high-water mark since the engine was built (reference: the session
        allocation categories and high-water of crates/sllm-core/src/execution.rs)."""
        def nbytes(t):
            return 0 if t is None else t.numel() * t.element_size()

        def weight_bytes(obj, seen, depth=0):
            total = 0
            if isinstance(obj, torch.Tensor):
                if obj.data_ptr() not in seen:
                    seen.add(obj.data_ptr())
                    total += nbytes(obj)
            elif isinstance(obj, (list, tuple)):
                total += sum(weight_bytes(x, seen, depth + 1) for x in obj)
            elif hasattr(obj, "__dict__") and depth < 6:
                total += sum(weight_bytes(v, seen, depth + 1) for v in vars(obj).values())
            return total

        cache = self.cache
        staging = sum(nbytes(getattr(self, n)) for n in ("d_tokens", "d_positions", "d_kv_lens", "d_seq_index", "d_table", "d_out",
                                                        "d_slots", "d_row_off", "d_rope_delta", "d_rope3", "d_logits"))
        pinned = sum(nbytes(getattr(self, n)) for n in ("h_tokens", "h_positions", "h_table", "h_out", "h_slots", "h_rope_delta"))
        out = {"weights": weight_bytes(self.model.w, set()),
               "kv_pages": nbytes(getattr(cache, "values", None)), "kv_scales": nbytes(getattr(cache, "scales", None)),
               "device_staging": staging, "pinned_host": pinned, "captured_graphs": len(self._graphs)}
        if self.is_cuda:
            ws = ops.workspace(self.device)
            out["kernel_workspace"] = sum(nbytes(getattr(ws, n, None)) for n in ("ws", "counters", "status"))
            out["allocator_now"] = torch.cuda.memory_allocated(self.device)
            out["allocator_high_water"] = torch.cuda.max_memory_allocated(self.device)
            out["allocator_at_build"] = self._mem_mark
        return out

    def kernel_timing(self, seqs: list) -> dict:
        """Runs ONE eager decode step of `seqs` with a CUDA event after every launch and returns the device time by
        launch kind: {"step_us", "launches", "by_kernel": {name: {"launches", "us"}}}.  The step is a real one (the
        sequences advance by a token); graphs are bypassed for it."""
        from ..ops import _lib
        self._guard()
        saved, self.use_graphs = self.use_graphs, False
        try:
            if self.is_cuda:
                torch.cuda.synchronize(self.device)
            _lib.timing(True)
            toks = self.decode(seqs)
            rep = _lib.timing_report()
        finally:
            _lib.timing(False)
            self.use_graphs = saved
        by: dict = {}
        for name, us in rep:
            e = by.setdefault(name, {"launches": 0, "us": 0.0})
            e["launches"] += 1
            e["us"] += us
        for e in by.values():
            e["us"] = round(e["us"], 2)
        for s_, t in zip(seqs, toks):
            s_.tokens.append(t)
        return {"step_us": round(sum(us for _, us in rep), 2), "launches": len(rep), "by_kernel": by}

    def embed_hidden(self, ids: list) -> torch.Tensor:
        """Final-normed hidden rows [len(ids), d] of one token list, computed on scratch KV pages that are released
        again (the embeddings / rerank endpoints pool these rows).  On a multi-rank engine the leader mirrors the call,
        so every rank runs the same kernels and collectives."""
        from .batch import make_prefill_batch
        from .. import ops
        self._guard()
        seq = self.new_sequence(ids)
        try:
            self.cache.pool.reserve(seq.seq_id, len(ids))
            table = torch.zeros((1, self.max_blocks), dtype=torch.int32)
            self.cache.pool.fill_block_table([seq.seq_id], table)
            b = make_prefill_batch([list(ids)], table.to(self.device), self.device, last_only=False)
            h = self.model.hidden(b, self.cache)
            return ops.rmsnorm(h, self.model.w.final_norm, self.cfg.rms_eps, self.cfg.norm_offset_one)
        finally:
            self.free_sequence(seq)

    def shutdown_report(self) -> dict:
        """What a supervisor logs when the engine goes away: memory by category, launch and copy counters, fallbacks
        and the quarantine record."""
        from ..ops import _lib
        return {"accounting": self.accounting(), "steps": self._steps, "kernel_launches": self.kernel_launches,
                "h2d_bytes": self.h2d_bytes, "d2h_bytes": self.d2h_bytes, "fallbacks": _lib.fallbacks(),
                "quarantine": self.quarantine,
                "kv_pool": self.cache.pool.stats() if hasattr(self.cache, "pool") else None}

    # ------------------------------------------------------------------ sequences
    def new_sequence(self, prompt: list, user=None) -> Sequence:
        self._guard()
        s = Sequence(prompt=list(prompt), user=user)
        s.seq_id = self.cache.pool.new_seq()
        if self.has_state:
            self.cache.alloc_slot(s.seq_id)
        return s

    def fork_sequence(self, src: Sequence, prompt: list, user=None) -> Sequence:
        """New sequence for `prompt` that reuses the KV of the longest common computed prefix of `src`
        (full pages shared by reference count, a partial last page copied).  At least one prompt token
        is left to compute so that the prefill produces logits."""
        limit = min(src.num_computed, len(prompt) - 1)
        common = 0
        while common < limit and src.tokens[common] == prompt[common]:
            common += 1
        if self.has_state and common != src.num_computed:
            common = 0        # a recurrent state describes the end of the source's computed tokens only
        s = Sequence(prompt=list(prompt), user=user)
        if common == 0:
            s.seq_id = self.cache.pool.new_seq()
            if self.has_state:
                self.cache.alloc_slot(s.seq_id)
        else:
            s.seq_id = self.cache.fork(src.seq_id, common)
            s.num_computed = common
            if self.has_state:
                self.cache.alloc_slot(s.seq_id)
                self.cache.copy_slot(src.seq_id, s.seq_id)
        return s

    def fork_kv(self, s: Sequence, n_tokens: int) -> int:
        """Pool-level fork (used by the prefix cache): a new pool sequence sharing the first `n_tokens` of `s`."""
        return self.cache.fork(s.seq_id, n_tokens)

    def free_kv(self, pool_seq_id: int) -> None:
        self.cache.pool.free_seq(pool_seq_id)

    def free_sequence(self, s: Sequence) -> None:
        if s.seq_id > 0:
            if self.has_state:
                self.cache.free_slot(s.seq_id)
            self.cache.pool.free_seq(s.seq_id)
            self._hidden_log.pop(s.seq_id, None)
            s.seq_id = -1

    def rollback(self, s: Sequence, length: int) -> None:
        """Speculative rollback / cancelled append: forget KV and tokens beyond ``length``."""
        if self.has_state and length < s.num_computed:
            raise ValueError("a recurrent-state model cannot rewind computed tokens without a state snapshot")
        self.cache.pool.truncate(s.seq_id, length)
        # the new tail may sit inside a page that a forked sibling or a prefix-cache entry still references: the next
        # append must not write into it (copy-on-write of the tail page)
        if hasattr(self.cache, "ensure_private_tail"):
            self.cache.ensure_private_tail(s.seq_id)
        s.num_computed = min(s.num_computed, length)
        del s.tokens[length:]
        log = self._hidden_log.get(s.seq_id)
        if log:
            kept = []
            for start, rows in log:
                if start < length:
                    kept.append((start, rows[:length - start]))
            self._hidden_log[s.seq_id] = kept

    def _rope3_rows(self, seqs: list, counts: list, positions: torch.Tensor) -> torch.Tensor:
        """3-axis rotary positions of text rows that follow a multimodal prompt: index + the sequence's delta."""
        delta = torch.tensor([s.rope_delta for s, c in zip(seqs, counts) for _ in range(c)], dtype=torch.int32,
                             device=positions.device)
        return (positions + delta).unsqueeze(0).expand(3, -1).contiguous()

    def _log_hidden(self, seqs: list, starts: list, counts: list, hidden: torch.Tensor) -> None:
        r0 = 0
        for s, st, n in zip(seqs, starts, counts):
            self._hidden_log.setdefault(s.seq_id, []).append((st, hidden[r0:r0 + n].clone()))
            r0 += n

    def hidden_start(self, s: Sequence) -> Optional[int]:
        """First position of ``s`` with a logged hidden row, or None."""
        log = self._hidden_log.get(s.seq_id)
        return log[0][0] if log else None

    def take_hidden(self, s: Sequence, start: int, end: int) -> torch.Tensor:
        """Logged hidden rows of positions [start, end) of ``s``; rows before ``end`` are dropped from the log."""
        log = self._hidden_log.get(s.seq_id, [])
        parts, rest, pos = [], [], start
        for st, rows in log:
            en = st + rows.shape[0]
            if en > pos and st <= pos < end:
                take = rows[pos - st:min(en, end) - st]
                parts.append(take)
                pos += take.shape[0]
            if en > end:
                rest.append((max(st, end), rows[max(st, end) - st:]))
        if pos != end:
            raise ValueError(f"hidden rows {pos}..{end} of sequence {s.seq_id} were not logged")
        self._hidden_log[s.seq_id] = rest
        return torch.cat(parts, 0) if len(parts) != 1 else parts[0]

    # ------------------------------------------------------------------ prefill
    def prefill(self, seqs: list, chunk_tokens: int = 0, sample: bool = True, embeds: Optional[torch.Tensor] = None,
                rope_pos3: Optional[torch.Tensor] = None, one_chunk: bool = False):
        """Runs the not-yet-computed prompt tokens of ``seqs``; returns greedy next tokens (list[int])
        or, with sample=False, the last-row logits [len(seqs), vocab].  A multimodal prompt passes ``embeds``
        ([T, d], the uncomputed tokens of all sequences in order, visual rows spliced in) and ``rope_pos3`` (int32
        [3, T]); it runs as one chunk and leaves each sequence's ``rope_delta`` for the decode steps.
        With ``one_chunk`` only the first ``chunk_tokens`` uncomputed tokens of every sequence run; a sequence is done
        when ``num_computed == len(tokens)`` afterwards, and only then is its row of the result meaningful (a
        scheduler interleaves the chunks of a long prompt with decode steps of the running requests)."""
        self._guard()
        if embeds is not None or rope_pos3 is not None:
            if chunk_tokens:
                raise ValueError("a multimodal prefill runs as one chunk")
            if rope_pos3 is not None and not self.cfg.mrope_sections:
                raise ValueError("the model has no multi-axis rotary sections")
        pool = self.cache.pool
        for s in seqs:
            pool.reserve(s.seq_id, len(s.tokens))
        table = torch.zeros((len(seqs), self.max_blocks), dtype=torch.int32)
        pool.fill_block_table([s.seq_id for s in seqs], table)
        d_table = table.to(self.device, non_blocking=True) if self.is_cuda else table
        self.h2d_bytes += table.numel() * 4
        starts = [s.num_computed for s in seqs]
        budget = chunk_tokens if chunk_tokens > 0 else max(len(s.tokens) for s in seqs)
        out = None
        while True:
            parts, part_starts, rows = [], [], []
            for i, s in enumerate(seqs):
                n = min(budget, len(s.tokens) - starts[i])
                if n > 0:
                    parts.append(s.tokens[starts[i]:starts[i] + n])
                    part_starts.append(starts[i])
                    rows.append(i)
            if not parts:
                break
            sub_table = d_table if len(rows) == len(seqs) else d_table[torch.tensor(rows, device=d_table.device)]
            b = make_prefill_batch(parts, sub_table, self.device, part_starts)
            if embeds is not None:
                b.embeds = embeds
            if rope_pos3 is not None:
                b.rope_pos3 = rope_pos3.to(self.device, torch.int32).contiguous()
                r0 = 0
                for j, i in enumerate(rows):
                    n_i = len(parts[j])
                    seqs[i].rope_delta = int(b.rope_pos3[:, r0:r0 + n_i].max().item()) + 1 - (part_starts[j] + n_i)
                    r0 += n_i
            elif self.cfg.mrope_sections and any(seqs[i].rope_delta for i in rows):
                b.rope_pos3 = self._rope3_rows([seqs[i] for i in rows], [len(p) for p in parts], b.positions)
            if self.has_state:
                b.slots = torch.tensor([self.cache.slot_of[seqs[i].seq_id] for i in rows], dtype=torch.int32, device=self.device)
            self.h2d_bytes += b.num_tokens * 12
            res = self.model.greedy(b, self.cache) if sample else self.model.forward(b, self.cache)
            if self.keep_hidden:
                self._log_hidden([seqs[i] for i in rows], part_starts, [len(p) for p in parts], self.model.last_hidden)
            if out is None:
                out = torch.zeros((len(seqs),) + tuple(res.shape[1:]), dtype=res.dtype, device=res.device)
            out[torch.tensor(rows, device=res.device)] = res
            for j, i in enumerate(rows):
                starts[i] += len(parts[j])
            if one_chunk and chunk_tokens > 0:
                break
        if sample:
            toks = out.tolist()
            self.d2h_bytes += 4 * len(seqs)
        self._table_key = None
        self._check_status(every=1)
        for i, s in enumerate(seqs):
            pool.commit(s.seq_id, starts[i])
            s.num_computed = starts[i]
        return toks if sample else out

    def extend(self, seqs: list, sample: bool = True, embeds: Optional[torch.Tensor] = None):
        """Runs every not-yet-computed token of each sequence as its own row (a speculative verify block, or
        any multi-token append) and returns, per sequence, the greedy token after each of those rows (or the
        logits [rows, vocab] with sample=False).  The block-table rows of one sequence are shared by its rows.
        ``embeds`` ([rows, d], in sequence order) replaces the embedding gather."""
        pool = self.cache.pool
        for s in seqs:
            pool.reserve(s.seq_id, len(s.tokens))
        table = torch.zeros((len(seqs), self.max_blocks), dtype=torch.int32)
        pool.fill_block_table([s.seq_id for s in seqs], table)
        d_table = table.to(self.device, non_blocking=True) if self.is_cuda else table
        parts = [s.tokens[s.num_computed:] for s in seqs]
        if any(not p for p in parts):
            raise ValueError("extend needs at least one uncomputed token per sequence")
        r = len(parts[0])
        if (sample and self.use_graphs and not self.has_state and embeds is None and r <= self.MAX_EXTEND_ROWS
                and not any(s.rope_delta for s in seqs)
                and len(seqs) <= self.max_batch and all(len(p) == r for p in parts)):
            return self._extend_graphed(seqs, parts, r, table)
        b = make_prefill_batch(parts, d_table, self.device, [s.num_computed for s in seqs], last_only=False)
        b.embeds = embeds
        if self.cfg.mrope_sections and any(s.rope_delta for s in seqs):
            b.rope_pos3 = self._rope3_rows(seqs, [len(p) for p in parts], b.positions)
        if self.has_state:
            b.slots = torch.tensor([self.cache.slot_of[s.seq_id] for s in seqs], dtype=torch.int32, device=self.device)
        self.h2d_bytes += table.numel() * 4 + b.num_tokens * 12
        res = self.model.greedy(b, self.cache) if sample else self.model.forward(b, self.cache)
        if self.keep_hidden:
            self._log_hidden(seqs, [s.num_computed for s in seqs], [len(p) for p in parts], self.model.last_hidden)
        self._table_key = None
        self._check_status(every=1)
        out, r0 = [], 0
        flat = res.tolist() if sample else None
        if sample:
            self.d2h_bytes += 4 * b.num_tokens
        for s, p in zip(seqs, parts):
            out.append(flat[r0:r0 + len(p)] if sample else res[r0:r0 + len(p)])
            r0 += len(p)
            pool.commit(s.seq_id, len(s.tokens))
            s.num_computed = len(s.tokens)
        return out

    MAX_EXTEND_ROWS = 9      # a verify block: the last committed token plus up to 8 drafts

    def _extend_graphed(self, seqs: list, parts: list, r: int, table: torch.Tensor):
        """`extend` for equally long blocks (speculative verify) replayed from a CUDA graph per (sequences, rows)."""
        n = len(seqs)
        t = n * r
        if getattr(self, "_ext", None) is None:
            cap = self.max_batch * self.MAX_EXTEND_ROWS
            pin = self.is_cuda
            self._ext = dict(
                h_tok=torch.zeros(cap, dtype=torch.int32, pin_memory=pin), h_pos=torch.zeros(cap, dtype=torch.int32, pin_memory=pin),
                d_tok=torch.zeros(cap, dtype=torch.int32, device=self.device), d_pos=torch.zeros(cap, dtype=torch.int32, device=self.device),
                d_kv=torch.ones(cap, dtype=torch.int32, device=self.device), d_out=torch.zeros(cap, dtype=torch.int32, device=self.device),
                h_out=torch.zeros(cap, dtype=torch.int32, pin_memory=pin), seq_index={}, graphs={}, launches={})
        e = self._ext
        flat_tok = [x for p in parts for x in p]
        flat_pos = [s.num_computed + i for s in seqs for i in range(r)]
        e["h_tok"][:t] = torch.tensor(flat_tok, dtype=torch.int32)
        e["h_pos"][:t] = torch.tensor(flat_pos, dtype=torch.int32)
        self.h_table[:n].copy_(table)
        self.d_table[:n].copy_(self.h_table[:n], non_blocking=True)
        self._table_key = None
        e["d_tok"][:t].copy_(e["h_tok"][:t], non_blocking=True)
        e["d_pos"][:t].copy_(e["h_pos"][:t], non_blocking=True)
        torch.add(e["d_pos"][:t], 1, out=e["d_kv"][:t])
        self.h2d_bytes += n * self.max_blocks * 4 + t * 8
        key = (n, r)
        si = e["seq_index"].get(key)
        if si is None:
            si = torch.arange(n, dtype=torch.int32, device=self.device).repeat_interleave(r).contiguous()
            e["seq_index"][key] = si

        def body():
            b = ForwardBatch(e["d_tok"][:t], e["d_pos"][:t], si, e["d_kv"][:t], self.d_table[:n], None, self.cfg.max_context)
            e["d_out"][:t] = self.model.greedy(b, self.cache)

        g = e["graphs"].get(key)
        if g is None:
            st = torch.cuda.Stream(device=self.device)
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                body()
            torch.cuda.current_stream().wait_stream(st)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            from ..ops import _lib
            before = _lib.LAUNCH_COUNT[0]
            with torch.cuda.graph(g):
                body()
            e["launches"][key] = _lib.LAUNCH_COUNT[0] - before
            e["graphs"][key] = g
            e.setdefault("hidden", {})[key] = self.model.last_hidden      # the graph's own output buffer
        g.replay()
        if self.keep_hidden:
            self._log_hidden(seqs, [s.num_computed for s in seqs], [r] * n, e["hidden"][key])
        self.kernel_launches += e["launches"][key]
        e["h_out"][:t].copy_(e["d_out"][:t], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += 4 * t
        flat = e["h_out"][:t].tolist()
        self._check_status()
        pool = self.cache.pool
        out = []
        for i, s in enumerate(seqs):
            out.append(flat[i * r:(i + 1) * r])
            pool.commit(s.seq_id, len(s.tokens))
            s.num_computed = len(s.tokens)
        return out

    # ------------------------------------------------------------------ decode
    def _decode_body(self, n: int, greedy: bool):
        b = ForwardBatch(self.d_tokens[:n], self.d_positions[:n], self.d_seq_index[:n], self.d_kv_lens[:n],
                         self.d_table[:n], None, self._max_kv)
        if self.has_state:
            b.row_off, b.slots = self.d_row_off[:n + 1], self.d_slots[:n]
        if self._rope3_on:
            b.rope_pos3 = self.d_rope3[:3 * n].view(3, n)
        if greedy:
            self.d_out[:n] = self.model.greedy(b, self.cache)
        else:
            lg = self.model.forward(b, self.cache)
            if self.d_logits is None or self.d_logits.shape[0] < self.max_batch:
                self.d_logits = torch.empty((self.max_batch, lg.shape[1]), dtype=lg.dtype, device=lg.device)
            self.d_logits[:n] = lg

    def _padded(self, n: int) -> int:
        if self.has_state:
            return n          # a padding row would advance row 0's recurrent state twice
        for g in self.GRAPH_BATCHES:
            if g >= n and g <= self.max_batch:
                return g
        return n

    def _run_decode(self, n: int, greedy: bool):
        if not self.use_graphs:
            self._decode_body(n, greedy)
            return
        key = (n, greedy, True) if self._rope3_on else (n, greedy)
        g = self._graphs.get(key)
        if g is None:
            # warm up outside capture (module init, workspace allocation), then capture
            # a recurrent state is advanced by every execution: keep it out of the warm-up run
            snap = (self.cache.conv_state.clone(), self.cache.rec_state.clone()) if self.has_state else None
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._decode_body(n, greedy)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            if snap is not None:
                self.cache.conv_state.copy_(snap[0])
                self.cache.rec_state.copy_(snap[1])
                torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            from ..ops import _lib
            before = _lib.LAUNCH_COUNT[0]
            with torch.cuda.graph(g):
                self._decode_body(n, greedy)
            self._graph_launches[key] = _lib.LAUNCH_COUNT[0] - before
            self._graphs[key] = g
        g.replay()
        self.kernel_launches += self._graph_launches[key]

    def warm_up(self, greedy_modes=(True, False)) -> int:
        """Captures the decode graphs of every padded batch size up front (a server would otherwise pay a
        capture, a few hundred milliseconds, the first time each batch size occurs).  Call while no sequence is
        live: the capture runs on the static input buffers.  Returns the number of graphs captured."""
        if not self.use_graphs or self.has_state:
            return 0
        made = 0
        self._rope3_on = False
        self._max_kv = self.cfg.max_context
        for n in self.GRAPH_BATCHES:
            if n > self.max_batch:
                break
            for greedy in greedy_modes:
                if (n, greedy) not in self._graphs:
                    self._run_decode(n, greedy)
                    made += 1
        torch.cuda.synchronize()
        return made

    def decode(self, seqs: list, sample: bool = True):
        """One token for every sequence (the last token of each is the input).  Returns greedy next
        tokens, or logits [len(seqs), vocab] with sample=False."""
        self._guard()
        n = len(seqs)
        if n > self.max_batch:
            raise ValueError("decode batch larger than max_batch")
        pool = self.cache.pool
        ps = self.cfg.page_size
        for s in seqs:
            pool.reserve(s.seq_id, len(s.tokens))
        np_ = self._padded(n)
        self.np_tokens[:n] = [s.tokens[-1] for s in seqs]
        self.np_positions[:n] = [len(s.tokens) - 1 for s in seqs]
        if np_ > n:  # padding rows replay row 0 (same token, same slot, same values: a harmless rewrite)
            self.np_tokens[n:np_] = self.np_tokens[0]
            self.np_positions[n:np_] = self.np_positions[0]
        # The block table changes only when a sequence crosses a page boundary or the batch changes.
        key = (tuple(s.seq_id for s in seqs), tuple((len(s.tokens) + ps - 1) // ps for s in seqs))
        if key != self._table_key:
            pool.fill_block_table([s.seq_id for s in seqs], self.h_table)
            if np_ > n:
                self.h_table[n:np_] = self.h_table[0]
            self.d_table[:np_].copy_(self.h_table[:np_], non_blocking=True)
            self.h2d_bytes += np_ * self.max_blocks * 4
            self._table_key = key
        self._max_kv = self.cfg.max_context
        if self.has_state:
            if np_ > n:
                raise ValueError("recurrent-state models decode unpadded batches only")
            self.h_slots[:n] = torch.tensor([self.cache.slot_of[s.seq_id] for s in seqs], dtype=torch.int32)
            self.d_slots[:n].copy_(self.h_slots[:n], non_blocking=True)
        self.d_tokens[:np_].copy_(self.h_tokens[:np_], non_blocking=True)
        self.d_positions[:np_].copy_(self.h_positions[:np_], non_blocking=True)
        torch.add(self.d_positions[:np_], 1, out=self.d_kv_lens[:np_])
        self.h2d_bytes += np_ * 8
        self._rope3_on = bool(self.cfg.mrope_sections) and any(s.rope_delta for s in seqs)
        if self._rope3_on:
            self.h_rope_delta[:n] = torch.tensor([s.rope_delta for s in seqs], dtype=torch.int32)
            if np_ > n:
                self.h_rope_delta[n:np_] = self.h_rope_delta[0]
            self.d_rope_delta[:np_].copy_(self.h_rope_delta[:np_], non_blocking=True)
            r3 = self.d_rope3[:3 * np_].view(3, np_)
            torch.add(self.d_positions[:np_], self.d_rope_delta[:np_], out=r3[0])
            r3[1].copy_(r3[0])
            r3[2].copy_(r3[0])
        self._run_decode(np_, sample)
        if sample:
            self.h_out[:np_].copy_(self.d_out[:np_], non_blocking=True)
            if self.is_cuda:
                torch.cuda.current_stream().synchronize()
            self.d2h_bytes += np_ * 4
            toks = self.h_out[:n].tolist()
        self._check_status()
        for s in seqs:
            pool.commit(s.seq_id, len(s.tokens))
            s.num_computed = len(s.tokens)
        return toks if sample else self.d_logits[:n]

    def _check_status(self, every: int = 64) -> None:
        self._steps += 1
        if self.is_cuda and (self._steps % every == 0 or every == 1):
            ws = ops.workspace(self.device)
            if int(ws.status[0].item()):
                code = ops.device_status(self.device)
                self._enter_quarantine(f"a bounded device wait gave up (status {code})", code)
                raise EngineQuarantined(f"device wait gave up (status {code}); the engine is quarantined")

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: list, max_new_tokens: int, eos: Optional[int] = None,
                 on_token: Optional[Callable] = None) -> list:
        """Greedy generation for a batch of prompts; returns the generated token lists."""
        seqs = [self.new_sequence(p) for p in prompts]
        try:
            first = self.prefill(seqs)
            done = [False] * len(seqs)
            for i, s in enumerate(seqs):
                s.tokens.append(first[i])
                if on_token:
                    on_token(i, first[i])
                if eos is not None and first[i] == eos:
                    done[i] = True
            for _ in range(max_new_tokens - 1):
                live = [s for i, s in enumerate(seqs) if not done[i]]
                if not live:
                    break
                toks = self.decode(live)
                k = 0
                for i, s in enumerate(seqs):
                    if done[i]:
                        continue
                    s.tokens.append(toks[k])
                    if on_token:
                        on_token(i, toks[k])
                    if eos is not None and toks[k] == eos:
                        done[i] = True
                    k += 1
            return [s.tokens[len(s.prompt):] for s in seqs]
        finally:
            for s in seqs:
                self.free_sequence(s)


def build_engine(cfg: ModelConfig, device="cuda", seed: int = 0, num_pages: Optional[int] = None,
                 max_batch: int = 64, use_cuda_graphs: bool = True, tp=None, ep=None) -> Engine:
    """Random-init engine for a named shape (benchmarks, tests, smoke).  `ep` (expert-parallel context) applies to
    the mixture-of-experts family and to hybrid models with a sparse MLP."""
    device = torch.device(device)
    tp_size, tp_rank = (tp.size, tp.rank) if tp is not None else (1, 0)
    if cfg.family == "qwen35":
        from ..cache.hybrid import HybridCache
        from ..models.qwen35 import Qwen35Model, init_random_qwen35_weights
        ep_size, ep_rank = (ep.size, ep.rank) if ep is not None else (1, 0)
        model = Qwen35Model(cfg, init_random_qwen35_weights(cfg, device, seed, tp_size=tp_size, tp_rank=tp_rank,
                                                            ep_size=ep_size, ep_rank=ep_rank), tp, ep)
        if num_pages is None:
            num_pages = max_batch * ((cfg.max_context + cfg.page_size - 1) // cfg.page_size) + 8
        cache = HybridCache(cfg, num_pages, device, max_seqs=2 * max_batch + 2, kv_heads=model.local_kv_heads,
                            tp_size=tp_size)
        return Engine(cfg, model, cache, device, max_batch=max_batch, use_cuda_graphs=use_cuda_graphs, tp=tp)
    if cfg.family == "moe":
        from ..models.moe import MoeModel, init_random_moe_weights
        ep_size, ep_rank = (ep.size, ep.rank) if ep is not None else (1, 0)
        weights = init_random_moe_weights(cfg, device, seed, tp_size, tp_rank, ep_size, ep_rank)
        model = MoeModel(cfg, weights, tp, ep)
    else:
        from ..models.llama import LlamaModel, init_random_weights
        weights = init_random_weights(cfg, device, seed, tp_size, tp_rank)
        model = LlamaModel(cfg, weights, tp)
    if num_pages is None:
        num_pages = max_batch * ((cfg.max_context + cfg.page_size - 1) // cfg.page_size) + 8
    cache = PagedKVCache(cfg, num_pages, device, kv_heads=model.local_kv_heads)
    return Engine(cfg, model, cache, device, max_batch=max_batch, use_cuda_graphs=use_cuda_graphs, tp=tp)

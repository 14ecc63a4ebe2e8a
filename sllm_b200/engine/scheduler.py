"""Continuous batching: a pure planning policy plus the loop that drives the engine with it.

`BatchPlanner` is the host-only policy of the reference's planner (crates/sllm-server/src/batching.rs:178-433):
waiting and decode-ready queues, compatibility classes (a Singleton lane never shares a step), bounded
round-robin decode rounds, one prefill admission after every `prefill_interval` decode rounds (or at
once when nothing is decoding), back-pressure (a request whose consumer is slow sits out rounds), and
deferred cancellation (a request in flight is cancelled when its round completes).  Unlike the
reference - where the planner is dead code because KV state is per-request scalar
(docs/plans/main-plan.md:894-904) - `EngineLoop` connects it to the GPU: every round is one call of
`Engine.prefill` / `Engine.decode` over per-row positions and block tables.

`EngineLoop` also carries the service-level behaviour of the reference's scheduler
(crates/sllm-server/src/runtime.rs:583-1137): bounded queue (`QueueFull` -> HTTP 429), slot registry
with queued / active / cancelled states, per-request timeout, drop-to-cancel, graceful drain.
"""
from __future__ import annotations

import collections
import itertools
import queue
import os
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Optional

import numpy as np

QUEUED, PREFILL_IN_FLIGHT, DECODE_READY, DECODE_IN_FLIGHT, BACKPRESSURED, FINISHED, CANCELLED, FAILED = (
    "queued", "prefill_in_flight", "decode_ready", "decode_in_flight", "backpressured", "finished", "cancelled",
    "failed")
TERMINAL = (FINISHED, CANCELLED, FAILED)
LANE_GREEDY, LANE_SAMPLED, LANE_SINGLETON = "dense_greedy", "dense_sampled", "singleton"


class PlannerError(RuntimeError):
    pass


class QueueFull(RuntimeError):
    pass


@dataclass
class _Entry:
    rid: int
    klass: tuple           # (model fingerprint, lane)
    phase: str = QUEUED
    cancel_requested: bool = False


@dataclass
class Round:
    kind: str              # "prefill" | "decode"
    rows: list             # request ids, row i = rows[i]


class BatchPlanner:
    def __init__(self, max_batch: int = 64, prefill_interval: int = 4, max_prefill_batch: int = 8):
        if max_batch < 1 or prefill_interval < 1 or max_prefill_batch < 1:
            raise PlannerError("invalid planner limits")
        self.max_batch, self.prefill_interval, self.max_prefill_batch = max_batch, prefill_interval, max_prefill_batch
        self.entries: dict = {}
        self.waiting: collections.deque = collections.deque()
        self.ready: collections.deque = collections.deque()
        self.in_flight: Optional[Round] = None
        self.decode_rounds_since_prefill = 0

    # ---------------------------------------------------------------- admission / cancellation
    def submit(self, rid: int, model: str, lane: str = LANE_GREEDY) -> None:
        if rid == 0 or rid in self.entries:
            raise PlannerError("request id must be non-zero and unique")
        if not model:
            raise PlannerError("empty compatibility identity")
        self.entries[rid] = _Entry(rid, (model, lane))
        self.waiting.append(rid)

    def cancel(self, rid: int) -> str:
        """Immediate for idle requests, deferred to round completion for in-flight ones."""
        e = self.entries.get(rid)
        if e is None or e.phase in TERMINAL:
            return e.phase if e else CANCELLED
        if e.phase in (PREFILL_IN_FLIGHT, DECODE_IN_FLIGHT):
            e.cancel_requested = True
            return e.phase
        self._remove_from_queues(rid)
        e.phase = CANCELLED
        return CANCELLED

    def _remove_from_queues(self, rid: int) -> None:
        for q in (self.waiting, self.ready):
            try:
                q.remove(rid)
            except ValueError:
                pass

    def phase(self, rid: int) -> str:
        return self.entries[rid].phase

    def forget(self, rid: int) -> None:
        e = self.entries.get(rid)
        if e is not None and e.phase in TERMINAL:
            del self.entries[rid]

    def set_backpressured(self, rid: int, on: bool) -> None:
        e = self.entries[rid]
        if on and e.phase == DECODE_READY:
            self.ready.remove(rid)
            e.phase = BACKPRESSURED
        elif not on and e.phase == BACKPRESSURED:
            e.phase = DECODE_READY
            self.ready.append(rid)

    # ---------------------------------------------------------------- rounds
    def next_round(self) -> Optional[Round]:
        if self.in_flight is not None:
            raise PlannerError("a round is already in flight")
        interval = 1 if getattr(self, "partial_prefill", False) else self.prefill_interval
        want_prefill = bool(self.waiting) and (not self.ready or self.decode_rounds_since_prefill >= interval)
        active = sum(1 for e in self.entries.values() if e.phase in (DECODE_READY, BACKPRESSURED))
        if want_prefill and active < self.max_batch:
            first = self.entries[self.waiting[0]]
            rows = []
            limit = 1 if first.klass[1] == LANE_SINGLETON else min(self.max_prefill_batch, self.max_batch - active)
            for rid in list(self.waiting):
                e = self.entries[rid]
                if e.klass[0] != first.klass[0] or (e.klass[1] == LANE_SINGLETON) != (first.klass[1] == LANE_SINGLETON):
                    continue
                rows.append(rid)
                if len(rows) >= limit:
                    break
            for rid in rows:
                self.waiting.remove(rid)
                self.entries[rid].phase = PREFILL_IN_FLIGHT
            self.decode_rounds_since_prefill = 0
            self.partial_prefill = False
            self.in_flight = Round("prefill", rows)
            return self.in_flight
        if self.ready:
            first = self.entries[self.ready[0]]
            limit = 1 if first.klass[1] == LANE_SINGLETON else self.max_batch
            rows = []
            for rid in list(self.ready):
                e = self.entries[rid]
                if e.klass[0] != first.klass[0] or (e.klass[1] == LANE_SINGLETON) != (first.klass[1] == LANE_SINGLETON):
                    continue
                rows.append(rid)
                if len(rows) >= limit:
                    break
            for rid in rows:
                self.ready.remove(rid)
                self.entries[rid].phase = DECODE_IN_FLIGHT
            self.decode_rounds_since_prefill += 1
            self.in_flight = Round("decode", rows)
            return self.in_flight
        return None

    def complete_round(self, outcomes: dict) -> list:
        """outcomes: rid -> "continue" | "finished" | "failed" | "backpressured".  Returns the ids whose
        deferred cancellation took effect."""
        rnd = self.in_flight
        if rnd is None:
            raise PlannerError("no round in flight")
        if set(outcomes) != set(rnd.rows):
            raise PlannerError("outcomes must cover exactly the rows of the round")
        cancelled = []
        for rid in rnd.rows:
            e = self.entries[rid]
            o = outcomes[rid]
            if o == "finished":
                e.phase = FINISHED
            elif o == "failed":
                e.phase = FAILED
            elif e.cancel_requested:
                e.phase = CANCELLED
                cancelled.append(rid)
            elif o == "backpressured":
                e.phase = BACKPRESSURED
            elif o == "prefill_more":
                # a long prompt ran one chunk: it goes back to the head of the waiting queue and its next chunk
                # follows after one decode round of the running requests
                e.phase = QUEUED
                self.waiting.insert(0, rid)
                self.partial_prefill = True
            elif o == "continue":
                e.phase = DECODE_READY
                self.ready.append(rid)       # round robin: back of the queue
            else:
                raise PlannerError(f"unknown outcome {o!r}")
        self.in_flight = None
        return cancelled

    def idle(self) -> bool:
        return self.in_flight is None and not self.waiting and not self.ready


# ------------------------------------------------------------------------------------------------
@dataclass
class GenRequest:
    """One generation job.  `on_token(token, selection)` returns False to stop; `on_done(reason)` is called
    exactly once with finish reason 'stop' | 'length' | 'cancelled' | 'error:<msg>' | 'timeout'."""
    prompt: list
    max_new_tokens: int
    chain: object = None                 # engine.sampling.SamplerChain or None (greedy)
    stop_tokens: tuple = ()
    on_token: Optional[Callable] = None
    on_done: Optional[Callable] = None
    mask_fn: Optional[Callable] = None   # () -> np.uint8[vocab] validity mask for the next token, or None
    deadline: Optional[float] = None
    singleton: bool = False
    rid: int = 0
    seq: object = None
    generated: int = 0
    state: str = "queued"                # queued | active | cancelled | done
    submitted_at: float = field(default_factory=time.monotonic)
    first_token_at: Optional[float] = None
    finish_reason: Optional[str] = None
    prefix_seq: object = None            # optional engine Sequence (or prefix-cache lease) whose KV prefix is forked
    prefix_hit_tokens: int = 0
    shifted_tokens: int = 0              # tokens dropped by context shifts so far
    shift_count: int = 0
    mm: object = None                    # multimodal prompt: mm(engine) -> (embeds [T, d], rope_pos3 [3, T])


class EngineLoop:
    """Single worker thread that owns the engine and runs planner rounds."""

    def __init__(self, engine, model_id: str = "model", max_batch: Optional[int] = None, queue_capacity: int = 64,
                 prefill_interval: int = 4, prefill_chunk_tokens: int = 0, prefix_cache=None, context_policy=None):
        self.engine = engine
        self.prefix_cache = prefix_cache
        self.context_policy = context_policy
        self.speculative = None              # engine.speculative.SpeculativeDecoder for greedy requests
        self.model_id = model_id
        self.planner = BatchPlanner(max_batch or engine.max_batch, prefill_interval,
                                    max_prefill_batch=min(8, max_batch or engine.max_batch))
        self.queue_capacity = queue_capacity
        self.prefill_chunk_tokens = prefill_chunk_tokens
        self.requests: dict = {}
        self._ids = itertools.count(1)
        self._lock = threading.Lock()
        self._wake = threading.Condition(self._lock)
        self._accepting = True
        self._stop = False
        self._calls: list = []               # (callable, result box) pairs to run on the engine thread between rounds
        self._thread = threading.Thread(target=self._run, name="sllm-engine-loop", daemon=True)
        self._thread.start()
        self.rounds = {"prefill": 0, "decode": 0}

    # ---------------------------------------------------------------- public
    def call(self, fn, timeout: float = 600.0):
        """Runs ``fn()`` on the engine thread between two rounds and returns its result (or raises what it raised).
        Device work and KV bookkeeping have one owner: a handler thread that needs the engine (embeddings, rerank) goes
        through here instead of touching it beside a running round - on a multi-rank engine that also keeps the
        mirrored commands in one order."""
        if threading.current_thread() is self._thread:
            return fn()
        box = {"done": threading.Event(), "out": None, "err": None}
        with self._wake:
            if self._stop:
                raise QueueFull("scheduler has stopped")
            self._calls.append((fn, box))
            self._wake.notify_all()
        if not box["done"].wait(timeout):
            raise TimeoutError("engine call timed out")
        if box["err"] is not None:
            raise box["err"]
        return box["out"]

    def submit(self, req: GenRequest) -> int:
        with self._wake:
            if not self._accepting:
                raise QueueFull("scheduler is draining")
            pending = sum(1 for r in self.requests.values() if r.state == "queued")
            if pending >= self.queue_capacity:
                raise QueueFull("queue is full")
            req.rid = next(self._ids)
            lane = LANE_SINGLETON if req.singleton else (LANE_GREEDY if req.chain is None else LANE_SAMPLED)
            self.requests[req.rid] = req
            self.planner.submit(req.rid, self.model_id, lane)
            self._wake.notify_all()
            return req.rid

    def cancel(self, rid: int) -> bool:
        with self._wake:
            req = self.requests.get(rid)
            if req is None or req.state == "done":
                return False
            phase = self.planner.cancel(rid)
            if phase == CANCELLED:
                self._finish(req, "cancelled")
            else:
                req.state = "cancelled"
            self._wake.notify_all()
            return True

    # Request audit: one record per finished request in a bounded ring (what was asked, what it cost, how it ended),
    # served by `/props`; the reference keeps the same per-request submission counts (include/sllm/hip.h:651-671).
    AUDIT_CAP = 128

    def _audit(self, req: GenRequest, reason: str) -> None:
        now = time.monotonic()
        rec = {"rid": req.rid, "prompt_tokens": len(req.prompt), "prefix_hit_tokens": req.prefix_hit_tokens,
               "generated": req.generated, "finish_reason": reason, "sampled": req.chain is not None,
               "constrained": req.mask_fn is not None, "multimodal": req.mm is not None,
               "context_shifts": req.shift_count, "shifted_tokens": req.shifted_tokens,
               "queue_to_first_token_ms": None if req.first_token_at is None
               else round((req.first_token_at - req.submitted_at) * 1e3, 3),
               "total_ms": round((now - req.submitted_at) * 1e3, 3),
               "decode_rounds_at_finish": self.rounds.get("decode", 0), "prefill_rounds_at_finish": self.rounds.get("prefill", 0)}
        ring = self.__dict__.setdefault("_audit_ring", [])
        ring.append(rec)
        if len(ring) > self.AUDIT_CAP:
            del ring[:len(ring) - self.AUDIT_CAP]

    def request_audit(self, n: int = 16) -> list:
        return list(self.__dict__.get("_audit_ring", []))[-n:]

    def slots(self) -> list:
        with self._lock:
            return [{"id": r.rid, "state": r.state, "phase": self.planner.entries[r.rid].phase
                     if r.rid in self.planner.entries else "done", "generated": r.generated,
                     "prompt_tokens": len(r.prompt)} for r in self.requests.values()]

    def stats(self) -> dict:
        with self._lock:
            states = collections.Counter(r.state for r in self.requests.values())
            return {"accepting": self._accepting, "queue_depth": states.get("queued", 0),
                    "active_requests": states.get("active", 0), "queue_capacity": self.queue_capacity,
                    "slots": self.planner.max_batch, "rounds": dict(self.rounds)}

    @property
    def accepting(self) -> bool:
        return self._accepting

    def shutdown(self, drain_timeout: float = 30.0) -> dict:
        """Stop accepting, let running requests finish until the timeout, cancel the rest."""
        with self._wake:
            self._accepting = False
            self._wake.notify_all()
        end = time.monotonic() + drain_timeout
        while time.monotonic() < end:
            with self._lock:
                if all(r.state == "done" for r in self.requests.values()):
                    break
            time.sleep(0.01)
        with self._wake:
            leftover = [r.rid for r in self.requests.values() if r.state != "done"]
        for rid in leftover:
            self.cancel(rid)
        with self._wake:
            self._stop = True
            self._wake.notify_all()
        self._thread.join(timeout=10)
        return {"cancelled_at_shutdown": len(leftover)}

    # ---------------------------------------------------------------- worker
    def _finish(self, req: GenRequest, reason: str) -> None:
        if req.state == "done":
            return
        req.state = "done"
        req.finish_reason = reason
        self._audit(req, reason)
        if req.prefix_seq is not None:
            self._release_prefix(req)
        if req.seq is not None:
            try:
                self.engine.free_sequence(req.seq)
            except Exception:
                pass
            req.seq = None
        if req.on_done:
            try:
                req.on_done(reason)
            except Exception:
                pass

    def _run(self) -> None:
        # SLLM_PROFILE_ENGINE_LOOP=<file>: cProfile statistics of this thread, written when the loop stops
        path = os.environ.get("SLLM_PROFILE_ENGINE_LOOP")
        if not path:
            return self._run_loop()
        import cProfile
        prof = cProfile.Profile()
        try:
            prof.runcall(self._run_loop)
        finally:
            prof.dump_stats(path)

    def _run_loop(self) -> None:
        while True:
            with self._wake:
                while not self._stop and self.planner.idle() and not self._calls:
                    self._wake.wait(timeout=0.05)
                    self._expire_locked()
                calls, self._calls = self._calls, []
                if self._stop:
                    for _, box in calls:
                        box["err"] = QueueFull("scheduler has stopped")
                        box["done"].set()
                    return
            for fn, box in calls:                  # outside the lock: submitters are not held up by device work
                try:
                    box["out"] = fn()
                except BaseException as exc:       # handed to the caller
                    box["err"] = exc
                finally:
                    box["done"].set()
            with self._wake:
                self._expire_locked()
                rnd = self.planner.next_round()
                if rnd is None:
                    continue
                reqs = [self.requests[rid] for rid in rnd.rows]
                for r in reqs:
                    if r.state == "queued":
                        r.state = "active"
            outcomes = self._execute(rnd.kind, reqs)
            with self._wake:
                self.rounds[rnd.kind] += 1
                cancelled = self.planner.complete_round(outcomes)
                for rid in cancelled:
                    self._finish(self.requests[rid], "cancelled")
                for r in reqs:
                    o = outcomes[r.rid]
                    if o in ("finished", "failed") and r.state != "done":
                        self._finish(r, r.finish_reason or ("stop" if o == "finished" else "error"))
                for rid in [rid for rid, r in self.requests.items() if r.state == "done"]:
                    self.planner.forget(rid)
                if len(self.requests) > 4 * self.queue_capacity + 256:
                    for rid in [rid for rid, r in self.requests.items() if r.state == "done"][:256]:
                        del self.requests[rid]

    def _expire_locked(self) -> None:
        now = time.monotonic()
        for r in list(self.requests.values()):
            if r.state in ("queued", "active") and r.deadline is not None and now > r.deadline:
                phase = self.planner.cancel(r.rid)
                r.finish_reason = "timeout"
                if phase == CANCELLED:
                    self._finish(r, "timeout")

    def _execute(self, kind: str, reqs: list) -> dict:
        eng = self.engine
        outcomes = {}
        try:
            if kind == "prefill":
                live = []
                for r in reqs:
                    if r.seq is not None:            # a later chunk of a prompt that is already under way
                        live.append(r)
                        continue
                    try:
                        if r.prefix_seq is not None:
                            try:
                                r.seq = eng.fork_sequence(r.prefix_seq, r.prompt)
                                r.prefix_hit_tokens = r.seq.num_computed
                            finally:
                                self._release_prefix(r)
                        else:
                            r.seq = eng.new_sequence(r.prompt)
                        live.append(r)
                    except Exception as exc:   # allocation failure poisons only this request
                        r.finish_reason = f"error:{type(exc).__name__}"
                        outcomes[r.rid] = "failed"
                plain = [r for r in live if r.mm is None]
                if plain:
                    chunked = self.prefill_chunk_tokens > 0
                    logits = eng.prefill([r.seq for r in plain], self.prefill_chunk_tokens, sample=False, one_chunk=chunked)
                    done = [i for i, r in enumerate(plain) if r.seq.num_computed == len(r.seq.tokens)]
                    for i, r in enumerate(plain):
                        if i not in done:
                            outcomes[r.rid] = "prefill_more"
                    fin = [plain[i] for i in done]
                    if fin:
                        if self.prefix_cache is not None:
                            for r in fin:
                                self.prefix_cache.publish(r.seq, len(r.prompt))
                        if len(fin) != len(plain):
                            import torch
                            logits = logits[torch.tensor(done, device=logits.device)]
                        self._select_and_publish(fin, logits, outcomes)
                for r in live:
                    if r.mm is None:
                        continue
                    # a multimodal prompt runs alone and in one chunk: visual rows replace the placeholder
                    # embeddings and the rotary positions carry three axes
                    try:
                        embeds, pos3 = r.mm(eng)
                        logits = eng.prefill([r.seq], sample=False, embeds=embeds, rope_pos3=pos3)
                    except Exception as exc:
                        r.finish_reason = f"error:{type(exc).__name__}:{exc}"
                        outcomes[r.rid] = "failed"
                        continue
                    self._select_and_publish([r], logits, outcomes)
            else:
                if self.context_policy is not None and not self.context_policy.is_disabled:
                    self._shift_full_windows(reqs)
                spec = [r for r in reqs if self.speculative is not None and r.chain is None and r.mask_fn is None]
                rest = [r for r in reqs if r not in spec]
                if spec:
                    self._speculative_round(spec, outcomes)
                if rest:
                    logits = eng.decode([r.seq for r in rest], sample=False)
                    self._select_and_publish(rest, logits, outcomes)
        except Exception as exc:
            for r in reqs:
                if r.rid not in outcomes:
                    r.finish_reason = f"error:{type(exc).__name__}:{exc}"
                    outcomes[r.rid] = "failed"
        return outcomes

    def _speculative_round(self, reqs: list, outcomes: dict) -> None:
        """Draft + verify for greedy requests; every accepted token goes through the same publication path."""
        budgets = [r.max_new_tokens - r.generated for r in reqs]
        new = self.speculative.step([r.seq for r in reqs], budgets)
        for r, toks in zip(reqs, new):
            del r.seq.tokens[len(r.seq.tokens) - len(toks):]      # re-appended one by one below
            for i, tok in enumerate(toks):
                self._publish_token(r, tok, None, outcomes)
                if outcomes[r.rid] != "continue":
                    # the request ended inside the block: forget the KV of the unpublished tail
                    if i + 1 < len(toks):
                        self.engine.rollback(r.seq, len(r.seq.tokens))
                    break
            if outcomes[r.rid] != "continue":
                self.speculative.release(r.seq)

    def _publish_token(self, r: GenRequest, tok: int, selection, outcomes: dict) -> None:
        if r.chain is not None:
            r.chain.accept(tok)
        r.seq.tokens.append(tok)
        r.generated += 1
        if r.first_token_at is None:
            r.first_token_at = time.monotonic()
        keep = True
        if r.on_token:
            keep = r.on_token(tok, selection) is not False
        if tok in r.stop_tokens:
            r.finish_reason = "stop"
            outcomes[r.rid] = "finished"
        elif not keep:
            r.finish_reason = r.finish_reason or "stop"
            outcomes[r.rid] = "finished"
        elif r.generated >= r.max_new_tokens:
            r.finish_reason = "length"
            outcomes[r.rid] = "finished"
        elif len(r.seq.tokens) >= self.engine.cfg.max_context and (
                self.context_policy is None or self.context_policy.is_disabled):
            r.finish_reason = "length"
            outcomes[r.rid] = "finished"
        else:
            outcomes[r.rid] = "continue"

    def _release_prefix(self, r: GenRequest) -> None:
        rel = getattr(r.prefix_seq, "release", None)
        r.prefix_seq = None
        if rel is not None:
            rel()

    def _shift_full_windows(self, reqs: list) -> None:
        """Compacts every sequence whose next token would fill the context (keep-prefix/keep-recent policy)."""
        from ..cache.context_shift import WindowState, apply_shift
        cap = self.engine.cfg.max_context
        for r in reqs:
            n = len(r.seq.tokens) - 1          # tokens held by the KV state; the last one is the decode input
            st = WindowState(n, n + r.shifted_tokens, r.shift_count)
            d = self.context_policy.plan(st, cap, 1)
            if d.shift:
                last = r.seq.tokens.pop()
                r.seq = apply_shift(self.engine, r.seq, d)
                r.seq.tokens.append(last)
                r.shifted_tokens += d.old_state.logical_length - d.new_state.logical_length
                r.shift_count += 1

    def _select_and_publish(self, reqs: list, logits, outcomes: dict) -> None:
        from .. import ops
        from . import sampling as S
        n = len(reqs)
        host_rows = [i for i, r in enumerate(reqs) if r.chain is not None or r.mask_fn is not None]
        host_logits = None
        device_rows = []
        if host_rows:
            device_rows = [i for i in host_rows if reqs[i].chain is not None and reqs[i].mask_fn is None
                           and logits.is_cuda and reqs[i].chain.supports_device_selector()
                           and not reqs[i].chain.cfg.logit_bias and not reqs[i].chain.counts_matter()]
        # the device argmax (a kernel and a synchronising read) only when some row needs it
        greedy_tokens = ops.argmax(logits).tolist() if logits.shape[0] and len(device_rows) < n else []
        if host_rows:
            dset = set(device_rows)
            need_host = [i for i in host_rows if i not in dset]
            if need_host:
                host_logits = {i: logits[i].float().cpu().numpy() for i in need_host}
        dev_tokens = {}
        if device_rows:
            import torch
            sel = logits if len(device_rows) == n else \
                logits[torch.tensor(device_rows, device=logits.device)].contiguous()
            recs = S.device_select(sel, [reqs[i].chain.device_row() for i in device_rows]).cpu().numpy() \
                .view(S.SELECTOR_RECORD_DTYPE).reshape(len(device_rows))
            for j, i in enumerate(device_rows):
                dev_tokens[i] = (int(recs["token"][j]), int(recs["status"][j]), float(recs["logprob"][j]))
        for i, r in enumerate(reqs):
            try:
                selection = None
                if i in dev_tokens:
                    tok, status, lp = dev_tokens[i]
                    if status != 0:
                        raise S.SamplingError("device selector: " + ("NaN logit" if status == 1 else "empty distribution"))
                    selection = S.Selection(tok, lp if r.chain.cfg.return_logprobs else None)
                elif r.chain is None and r.mask_fn is None:
                    tok = greedy_tokens[i]
                    if tok < 0:
                        raise S.SamplingError("NaN logit")
                else:
                    mask = r.mask_fn() if r.mask_fn is not None else None
                    chain = r.chain or S.SamplerChain(S.SamplerChainConfig())
                    selection = chain.select(host_logits[i], device_argmax=greedy_tokens[i], valid_mask=mask)
                    tok = selection.token
                self._publish_token(r, tok, selection, outcomes)
            except Exception as exc:
                r.finish_reason = f"error:{type(exc).__name__}:{exc}"
                outcomes[r.rid] = "failed"

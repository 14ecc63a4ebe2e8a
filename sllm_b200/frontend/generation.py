"""Transport-independent generation service: tokens in, visible text deltas out.

The per-request loop of the reference (crates/sllm-frontend/src/generation.rs:2125-2503) - sampler chain,
grammar / EOS / reasoning masks, stop tokens, incremental detokenisation with UTF-8 hold-back, stop-string
matching, usage accounting - runs here as callbacks of one `GenRequest` inside the continuous-batching
`EngineLoop`, so many requests share every GPU step.  Consumers read an event queue:
    ("delta", {"content": str, "reasoning": str, "tokens": [...], "logprobs": [...]})
    ("done",  {"finish_reason": "stop" | "length" | "cancelled" | "timeout" | "error", "usage": {...}, "error": str?})
The queue is bounded: a slow consumer back-pressures only its own request (runtime.rs:701-705 drop-to-cancel is
`GenerationHandle.cancel`).
"""
from __future__ import annotations

import collections
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Optional

from ..engine import sampling as S
from ..engine.scheduler import EngineLoop, GenRequest, QueueFull
from .reasoning import ReasoningController, ReasoningSeparator
from .text import IncrementalDetokenizer, IncrementalStopMatcher, TokenByteTable

MAX_COMPLETION_TOKENS = 4096


@dataclass
class GenerationConfig:
    max_new_tokens: int = 256
    chain: S.SamplerChainConfig = field(default_factory=S.SamplerChainConfig)
    seed: Optional[int] = None
    stop: tuple = ()
    thinking: bool = False
    separate_reasoning: bool = False
    reasoning_budget: Optional[int] = None
    grammar_gbnf: Optional[str] = None
    assistant_prefill: str = ""
    timeout_s: Optional[float] = None
    ignore_eos: bool = False
    echo_tokens: bool = False


class _LoopNotifier:
    """One wake-up of an asyncio loop for any number of channels that became readable: producers (the engine thread)
    post a channel; the first post since the last flush schedules ONE `call_soon_threadsafe`, the flush wakes every
    posted channel's waiter.  An engine round that publishes a token for each of 32 streams thus costs one self-pipe
    write instead of 32 thread hand-offs."""

    _by_loop: dict = {}
    _guard = threading.Lock()

    def __init__(self, loop):
        self.loop = loop
        self._lock = threading.Lock()
        self._ready: list = []
        self._scheduled = False

    @classmethod
    def of(cls, loop) -> "_LoopNotifier":
        with cls._guard:
            n = cls._by_loop.get(id(loop))
            if n is None or n.loop is not loop:
                if len(cls._by_loop) > 64:
                    cls._by_loop.clear()
                n = cls._by_loop[id(loop)] = _LoopNotifier(loop)
            return n

    def post(self, channel: "EventChannel") -> None:
        with self._lock:
            self._ready.append(channel)
            if self._scheduled:
                return
            self._scheduled = True
        try:
            self.loop.call_soon_threadsafe(self._flush)
        except RuntimeError:                 # the loop is closed: nobody is waiting any more
            with self._lock:
                self._scheduled = False
                self._ready.clear()

    def _flush(self) -> None:
        with self._lock:
            ready, self._ready = self._ready, []
            self._scheduled = False
        for ch in ready:
            ch._wake_async()


class EventChannel:
    """Bounded event queue between the engine thread (producer) and one consumer that is either a thread (`get`,
    iteration) or a coroutine (`aget`, `aget_batch`).  The coroutine side needs no helper thread: it parks a future,
    and the producer wakes the loop through the loop's notifier only while such a future is parked.  Same exceptions
    as queue.Queue (queue.Full / queue.Empty)."""

    def __init__(self, capacity: int):
        self.capacity = capacity
        self._items: collections.deque = collections.deque()
        self._cv = threading.Condition(threading.Lock())
        self._waiter = None              # asyncio.Future of the coroutine consumer, owned by its loop
        self._notifier: Optional[_LoopNotifier] = None

    # ---- producer
    def put(self, item, timeout: Optional[float] = None) -> None:
        with self._cv:
            if len(self._items) >= self.capacity:
                if not self._cv.wait_for(lambda: len(self._items) < self.capacity, timeout):
                    raise queue.Full
            self._items.append(item)
            self._cv.notify()
            notifier = self._notifier if self._waiter is not None else None
        if notifier is not None:
            notifier.post(self)

    def put_nowait(self, item) -> None:
        with self._cv:
            if len(self._items) >= self.capacity:
                raise queue.Full
            self._items.append(item)
            self._cv.notify()
            notifier = self._notifier if self._waiter is not None else None
        if notifier is not None:
            notifier.post(self)

    # ---- thread consumer
    def get(self, timeout: Optional[float] = None):
        with self._cv:
            if not self._cv.wait_for(lambda: self._items, timeout):
                raise queue.Empty
            item = self._items.popleft()
            self._cv.notify()
            return item

    def get_nowait(self):
        with self._cv:
            if not self._items:
                raise queue.Empty
            item = self._items.popleft()
            self._cv.notify()
            return item

    def qsize(self) -> int:
        return len(self._items)

    # ---- coroutine consumer (one at a time)
    def _wake_async(self) -> None:
        with self._cv:
            w, self._waiter = self._waiter, None
        if w is not None and not w.done():
            w.set_result(None)

    async def aget_batch(self, limit: int = 64) -> list:
        """Waits for one event, then takes what else is queued (up to `limit`, stopping after a terminal event)."""
        import asyncio
        loop = asyncio.get_running_loop()
        while True:
            with self._cv:
                if self._items:
                    out = [self._items.popleft()]
                    while len(out) < limit and out[-1][0] == "delta" and self._items:
                        out.append(self._items.popleft())
                    self._cv.notify_all()
                    return out
                self._notifier = _LoopNotifier.of(loop)
                self._waiter = fut = loop.create_future()
            try:
                await fut
            finally:
                with self._cv:
                    if self._waiter is fut:
                        self._waiter = None

    async def aget(self):
        return (await self.aget_batch(1))[0]


class GenerationHandle:
    def __init__(self, service: "GenerationService", capacity: int):
        self.events: EventChannel = EventChannel(capacity)
        self.service = service
        self.rid = 0
        self.prompt_tokens = 0
        self.completion_tokens = 0
        self.finish_reason: Optional[str] = None
        self._done = threading.Event()

    def cancel(self) -> None:
        if self.rid:
            self.service.loop.cancel(self.rid)

    def wait(self, timeout: Optional[float] = None) -> bool:
        return self._done.wait(timeout)

    def __iter__(self):
        while True:
            kind, payload = self.events.get()
            yield kind, payload
            if kind == "done":
                return

    def collect(self):
        """Blocks until done; returns (content, reasoning, done payload)."""
        content, reasoning, done = [], [], None
        for kind, payload in self:
            if kind == "delta":
                content.append(payload.get("content", ""))
                reasoning.append(payload.get("reasoning", ""))
            else:
                done = payload
        return "".join(content), "".join(reasoning), done


class GenerationService:
    def __init__(self, loop: EngineLoop, tokenizer, vocab_size: int, model_id: str = "model", event_capacity: int = 256):
        self.loop = loop
        self.tk = tokenizer
        self.vocab = vocab_size
        self.model_id = model_id
        self.event_capacity = event_capacity
        self._byte_table: Optional[TokenByteTable] = None
        self._grammar_cache: dict = {}
        self._lock = threading.Lock()

    # ------------------------------------------------------------------------------------------
    def byte_table(self) -> list:
        with self._lock:
            if self._byte_table is None:
                self._byte_table = TokenByteTable(self.tk, self.vocab)
            return self._byte_table.bytes

    def _grammar(self, gbnf: str):
        from ..engine.grammar import CompiledGrammar
        with self._lock:
            g = self._grammar_cache.get(gbnf)
        if g is None:
            g = CompiledGrammar(gbnf, self.byte_table())
            with self._lock:
                if len(self._grammar_cache) > 32:
                    self._grammar_cache.clear()
                self._grammar_cache[gbnf] = g
        return g

    def submit(self, prompt_ids: list, cfg: GenerationConfig, prefix_seq=None, mm=None) -> GenerationHandle:
        """``mm`` (models.vision_tower.MultimodalPrompt) marks a prompt with images: ``prompt_ids`` must then be
        its expanded token list."""
        if not prompt_ids:
            raise ValueError("prompt must contain at least one token")
        if not 1 <= cfg.max_new_tokens <= MAX_COMPLETION_TOKENS:
            raise ValueError("max_new_tokens must be in 1..4096")
        if len(prompt_ids) + cfg.max_new_tokens > self.loop.engine.cfg.max_context:
            raise ValueError("prompt plus max_new_tokens exceeds the server context length")
        h = GenerationHandle(self, self.event_capacity)
        h.prompt_tokens = len(prompt_ids)
        eos_ids = tuple(getattr(self.tk, "eos_ids", ()) or ())
        chain_cfg = cfg.chain
        needs_chain = chain_cfg.requires_logits or chain_cfg.extended or chain_cfg.ignore_eos_token is not None
        chain = S.SamplerChain(chain_cfg, prompt_ids if (chain_cfg.extended or chain_cfg.params.frequency_penalty
                                                         or chain_cfg.params.presence_penalty) else (), seed=cfg.seed) \
            if needs_chain else None
        detok = IncrementalDetokenizer(self.tk, skip_special_tokens=True)
        stopper = IncrementalStopMatcher(list(cfg.stop)) if cfg.stop else None
        separator = ReasoningSeparator(starts_in_reasoning=cfg.thinking) if cfg.separate_reasoning else None
        gstate = None
        if cfg.grammar_gbnf:
            gstate = self._grammar(cfg.grammar_gbnf).new_state()
            if cfg.assistant_prefill and not gstate.accept_text(cfg.assistant_prefill):
                raise ValueError("assistant prefill is not a prefix of the requested grammar")
        rctl = None
        if cfg.thinking and cfg.reasoning_budget:
            close_ids = self.tk.encode("</think>")
            rctl = ReasoningController(cfg.reasoning_budget, close_ids, self.vocab)
        state = {"stopped_by_string": False, "logprobs": []}

        def mask_fn():
            m = None
            if rctl is not None:
                m = rctl.mask()
            if m is None and gstate is not None and (rctl is None or not rctl.active):
                m = gstate.mask(eos_ids=eos_ids)
            return m

        def publish(content: str, reasoning: str, token: int, sel) -> bool:
            payload = {"content": content, "reasoning": reasoning}
            if cfg.echo_tokens:
                payload["tokens"] = [token]
            if sel is not None and sel.logprob is not None:
                payload["logprobs"] = [{"token": token, "logprob": sel.logprob, "top": sel.top_logprobs}]
            if not (content or reasoning or "logprobs" in payload or cfg.echo_tokens):
                return True
            try:
                h.events.put(("delta", payload), timeout=30.0)
                return True
            except queue.Full:
                return False      # consumer is gone or stuck: stop this request

        def on_token(tok: int, sel) -> bool:
            h.completion_tokens += 1
            if rctl is not None:
                rctl.accept(tok)
            if gstate is not None and (rctl is None or not rctl.active) and tok not in eos_ids:
                gstate.accept(tok)
            if tok in eos_ids and not cfg.ignore_eos:
                return True           # stop_tokens ends the request; nothing to publish
            text = detok.push(tok)
            stop_now = False
            if stopper is not None:
                text, stop_now = stopper.push(text)
            reasoning = ""
            if separator is not None:
                reasoning, text = separator.push(text)
            ok = publish(text, reasoning, tok, sel)
            if stop_now:
                state["stopped_by_string"] = True
                return False
            return ok

        def on_done(reason: str) -> None:
            tail = detok.flush()
            if stopper is not None and not state["stopped_by_string"]:
                tail, _ = stopper.push(tail)
                tail += stopper.flush()
            elif state["stopped_by_string"]:
                tail = ""
            reasoning = ""
            if separator is not None:
                r1, tail = separator.push(tail)
                r2, t2 = separator.flush()
                reasoning, tail = r1 + r2, tail + t2
            if (tail or reasoning) and not reason.startswith("error") and reason not in ("cancelled", "timeout"):
                try:
                    h.events.put_nowait(("delta", {"content": tail, "reasoning": reasoning}))
                except queue.Full:
                    pass
            err = None
            if reason.startswith("error"):
                err, reason = reason[6:] or "generation failed", "error"
            h.finish_reason = reason
            payload = {"finish_reason": reason,
                       "usage": {"prompt_tokens": h.prompt_tokens, "completion_tokens": h.completion_tokens,
                                 "total_tokens": h.prompt_tokens + h.completion_tokens}}
            if err:
                payload["error"] = err
            while True:
                try:
                    h.events.put_nowait(("done", payload))
                    break
                except queue.Full:
                    try:
                        h.events.get_nowait()      # the terminal event must fit; drop the oldest delta
                    except queue.Empty:
                        pass
            h._done.set()

        req = GenRequest(prompt=list(prompt_ids), max_new_tokens=cfg.max_new_tokens, chain=chain,
                         stop_tokens=() if cfg.ignore_eos else eos_ids, on_token=on_token, on_done=on_done,
                         mask_fn=mask_fn if (gstate is not None or rctl is not None) else None,
                         deadline=(time.monotonic() + cfg.timeout_s) if cfg.timeout_s else None,
                         prefix_seq=None if mm is not None else prefix_seq, mm=mm)
        h.rid = self.loop.submit(req)
        h.request = req
        return h

    def generate_text(self, prompt: str, cfg: GenerationConfig):
        """Convenience: tokenise, run to completion, return (text, reasoning, done payload)."""
        ids = self.tk.encode(prompt)
        return self.submit(ids, cfg).collect()

"""Generation backends behind the HTTP service.

`EngineBackend` is the production backend: resident weights, paged KV cache, continuous-batching loop,
generation service, prefix cache and embeddings - the counterpart of the reference's `QwenChatBackendV1`
(crates/sllm-server/src/production.rs:2544,3513,3583) minus its whole-generation mutex: requests share GPU steps.
The scripted backends reproduce the reference's HTTP contract-test doubles
(crates/sllm-server/tests/http_contract.rs:26-138): Script, Blocking, Endless, FailOnce.
"""
from __future__ import annotations

import queue
import threading
import time
from typing import Optional

import numpy as np

from ..engine.scheduler import QueueFull
from ..frontend.generation import EventChannel, GenerationConfig, GenerationHandle, GenerationService
from ..frontend.text import ByteTokenizer


class ScriptHandle:
    def __init__(self, prompt_tokens: int):
        self.events = EventChannel(1 << 20)
        self.prompt_tokens = prompt_tokens
        self.completion_tokens = 0
        self.cancelled = threading.Event()
        self.rid = 0

    def cancel(self):
        self.cancelled.set()

    def __iter__(self):
        while True:
            kind, payload = self.events.get()
            yield kind, payload
            if kind == "done":
                return


class ScriptBackend:
    """Emits a fixed list of deltas (optionally (content, reasoning) tuples) and a finish reason."""

    def __init__(self, deltas=("Hello", ", ", "world"), finish_reason="stop", aliases=("test-model",), delay: float = 0.0,
                 queue_capacity: int = 8):
        self.aliases = list(aliases)
        self.deltas, self.finish_reason, self.delay = list(deltas), finish_reason, delay
        self.tokenizer = ByteTokenizer()
        self.accepting = True
        self.queue_capacity = queue_capacity
        self.active = 0
        self._lock = threading.Lock()
        self.handles: dict = {}
        self._next = 1
        self.submitted = []

    # --- service surface
    def props(self) -> dict:
        return {"backend": type(self).__name__, "context_length": 4096, "kv_cache_encoding": "none", "vocab_size": self.tokenizer.vocab_size}

    def memory(self) -> dict:
        return {"weights": 0, "kv_cache": 0, "workspace": 0}

    def scheduler_stats(self) -> dict:
        return {"accepting": self.accepting, "active_requests": self.active, "queue_capacity": self.queue_capacity,
                "queue_depth": 0, "slots": 1}

    def slots(self) -> list:
        with self._lock:
            return [{"id": i, "state": "active", "generated": h.completion_tokens, "prompt_tokens": h.prompt_tokens}
                    for i, h in self.handles.items()]

    def cancel_slot(self, sid: int) -> bool:
        with self._lock:
            h = self.handles.get(sid)
        if h is None:
            return False
        h.cancel()
        return True

    def max_context(self) -> int:
        return 4096

    def embed(self, token_lists: list) -> list:
        out = []
        for ids in token_lists:
            v = np.zeros(8, dtype=np.float64)
            for i, t in enumerate(ids):
                v[(t + i) % 8] += 1.0
            n = np.linalg.norm(v)
            out.append((v / n if n > 0 else v).astype(np.float32))
        return out

    def shutdown(self, timeout: float = 5.0) -> dict:
        self.accepting = False
        return {"cancelled_at_shutdown": 0}

    # --- generation
    def _register(self, h: ScriptHandle):
        with self._lock:
            if not self.accepting or self.active >= self.queue_capacity:
                raise QueueFull("queue is full")
            h.rid = self._next
            self._next += 1
            self.handles[h.rid] = h
            self.active += 1

    def _finish(self, h: ScriptHandle, reason: str, error: Optional[str] = None):
        payload = {"finish_reason": reason, "usage": {"prompt_tokens": h.prompt_tokens,
                                                      "completion_tokens": h.completion_tokens,
                                                      "total_tokens": h.prompt_tokens + h.completion_tokens}}
        if error:
            payload["error"] = error
        h.events.put(("done", payload))
        with self._lock:
            self.handles.pop(h.rid, None)
            self.active -= 1

    def submit(self, prompt_ids: list, cfg: GenerationConfig, prefix_seq=None) -> ScriptHandle:
        h = ScriptHandle(len(prompt_ids))
        self._register(h)
        self.submitted.append((list(prompt_ids), cfg))
        threading.Thread(target=self._run, args=(h, cfg), daemon=True).start()
        return h

    def _run(self, h: ScriptHandle, cfg: GenerationConfig):
        for d in self.deltas:
            if h.cancelled.is_set():
                return self._finish(h, "cancelled")
            if self.delay:
                time.sleep(self.delay)
            content, reasoning = (d, "") if isinstance(d, str) else d
            h.completion_tokens += 1
            h.events.put(("delta", {"content": content, "reasoning": reasoning}))
            if h.completion_tokens >= cfg.max_new_tokens:
                return self._finish(h, "length")
        self._finish(h, self.finish_reason)


class BlockingBackend(ScriptBackend):
    """Produces nothing until `release` is set or the request is cancelled."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.release = threading.Event()

    def _run(self, h, cfg):
        while not self.release.is_set():
            if h.cancelled.wait(0.01):
                return self._finish(h, "cancelled")
        super()._run(h, cfg)


class EndlessBackend(ScriptBackend):
    def _run(self, h, cfg):
        while not h.cancelled.is_set():
            h.completion_tokens += 1
            h.events.put(("delta", {"content": "x", "reasoning": ""}))
            if h.completion_tokens >= cfg.max_new_tokens:
                return self._finish(h, "length")
            time.sleep(0.002)
        self._finish(h, "cancelled")


class FailOnceBackend(ScriptBackend):
    """The first request fails after one delta; later requests succeed."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.failed = False

    def _run(self, h, cfg):
        if not self.failed:
            self.failed = True
            h.completion_tokens += 1
            h.events.put(("delta", {"content": "partial", "reasoning": ""}))
            return self._finish(h, "error", "backend failure")
        super()._run(h, cfg)


class EngineBackend:
    """Engine + continuous-batching loop + generation service for one resident model."""

    def __init__(self, engine, tokenizer, aliases=("model",), queue_capacity: int = 64, event_capacity: int = 256,
                 prefill_chunk_tokens: int = 0, prefix_cache=None, kv_cache_encoding: str = "bf16",
                 context_policy=None, checkpoint_store=None):
        from ..engine.scheduler import EngineLoop
        self.engine = engine
        self.tokenizer = tokenizer
        self.aliases = list(aliases)
        if prefix_cache is True:
            from ..cache.prefix import PrefixCache, PrefixIdentity
            prefix_cache = PrefixCache(engine, PrefixIdentity(
                model=engine.cfg.name, tokenizer=getattr(tokenizer, "identity", type(tokenizer).__name__),
                kv_layout=engine.cfg.kv_format, context_policy=context_policy.identity() if context_policy else ""))
        self.prefix_cache = prefix_cache or None
        self.context_policy = context_policy
        self.checkpoint_store = checkpoint_store
        self.loop = EngineLoop(engine, self.aliases[0], queue_capacity=queue_capacity,
                               prefill_chunk_tokens=prefill_chunk_tokens, prefix_cache=self.prefix_cache,
                               context_policy=context_policy)
        self.service = GenerationService(self.loop, tokenizer, engine.cfg.vocab, self.aliases[0], event_capacity)
        self.kv_cache_encoding = kv_cache_encoding
        self._embed_lock = threading.Lock()

    @property
    def accepting(self) -> bool:
        return self.loop.accepting and getattr(self.engine, "quarantine", None) is None

    def props(self) -> dict:
        c = self.engine.cfg
        from ..ops import w4 as _w4
        return {"backend": "sllm-b200", "quarantine": getattr(self.engine, "quarantine", None), "model_family": c.family,
                "activation_encoding": "fp4" if _w4.w4a4_enabled() else "bf16", "context_length": c.max_context, "vocab_size": c.vocab,
                "kv_cache_encoding": c.kv_format, "weight_format": c.weight_format, "page_size": c.page_size,
                "tensor_parallel": getattr(self.engine.tp, "size", 1) if self.engine.tp else 1,
                "prefix_cache": self.prefix_cache is not None, "vision": getattr(self.engine, "vision", None) is not None}

    def memory(self) -> dict:
        cache = self.engine.cache
        kv = cache.values.numel() * cache.values.element_size() + (cache.scales.numel() * 4 if cache.scales is not None else 0)
        w = 0
        try:
            ws = self.engine.model.w
            tensors = [ws.embed, ws.final_norm, ws.lm_head.w] + [t for l in ws.layers for t in (l.qkv.w, l.o.w, l.gate_up.w, l.down.w)]
            w = sum(t.numel() * t.element_size() for t in tensors)
        except Exception:
            pass
        return {"weights": w, "kv_cache": kv, "kv_pages_free": cache.pool.stats()["free"] * cache.bytes_per_token() * cache.spec.page_size}

    def scheduler_stats(self) -> dict:
        return self.loop.stats()

    def request_audit(self, n: int = 16) -> list:
        return self.loop.request_audit(n)

    def slots(self) -> list:
        return self.loop.slots()

    def cancel_slot(self, sid: int) -> bool:
        return self.loop.cancel(sid)

    def max_context(self) -> int:
        return self.engine.cfg.max_context

    def submit(self, prompt_ids: list, cfg: GenerationConfig, prefix_seq=None, mm=None) -> GenerationHandle:
        if mm is not None:                       # prompts with images bypass the (token-keyed) prefix cache
            return self.service.submit(prompt_ids, cfg, mm=mm)
        if prefix_seq is None and self.prefix_cache is not None:
            prefix_seq = self.prefix_cache.lookup(prompt_ids)
        return self.service.submit(prompt_ids, cfg, prefix_seq=prefix_seq)

    def multimodal_prompt(self, text: str, images: list):
        """Tokenises a rendered prompt whose image markers stand for `images` (frontend.vision.BoundedImage) and
        returns the models.vision_tower.MultimodalPrompt for `submit`."""
        from ..frontend import vision as V
        from ..models.vision_tower import MultimodalPrompt, encode_with_images
        tower = getattr(self.engine, "vision", None)
        if tower is None:
            raise ValueError("the model has no vision tower")
        tok_id = self.engine.cfg.image_token_id
        if tok_id is None:
            tok_id = self.engine.cfg.vocab - 1
        return MultimodalPrompt(tower, V.process_many(images), encode_with_images(self.tokenizer, text, tok_id), tok_id)

    def embed(self, token_lists: list) -> list:
        """Mean of the final hidden rows in float64, L2-normalised, finite float32
        (reference: crates/sllm-core/src/inference_embedding.rs)."""
        import torch

        def one(ids):
            h = self.engine.embed_hidden(ids)
            v = h.double().mean(dim=0)
            n = torch.linalg.vector_norm(v)
            v = (v / n if float(n) > 0 else v).float().cpu().numpy()
            if not np.isfinite(v).all():
                raise ValueError("embedding is not finite")
            return v

        # one list per engine call: generation rounds of other requests interleave with a long batch of inputs
        with self._embed_lock:
            return [self.loop.call(lambda ids=ids: one(ids)) for ids in token_lists]

    def shutdown(self, timeout: float = 30.0) -> dict:
        return self.loop.shutdown(timeout)

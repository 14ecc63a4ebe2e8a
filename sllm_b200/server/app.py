"""HTTP service: every route, status code and SSE framing of the reference's router
(crates/sllm-server/src/service.rs:179-213,251-293), on FastAPI / Starlette.

Routes: /healthz /readyz /metrics /props /slots /admin/slots/{id}/cancel /admin/keys/reload
/admin/models/{alias}/{load,preload,unload,clear-quarantine} /admin/models/evict-idle /v1/models
/v1/chat/completions (+ /{id}/events) /v1/completions /v1/embeddings /v1/rerank /v1/infill /v1/tokenize
/v1/detokenize /v1/apply-template /v1/input-tokens /v1/responses (+ /{id}/events) /v1/messages (+ /{id}/events).
"""
from __future__ import annotations

import asyncio
import base64
import json
import time
import uuid
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse, Response, StreamingResponse

from ..engine.grammar import JSON_OBJECT_GBNF, GrammarError, schema_to_gbnf
from ..engine.sampling import derive_choice_seed
from ..engine.scheduler import QueueFull
from ..frontend import tools as T
from ..frontend.chat import ChatMessage, ChatRenderError, render_chatml, render_infill
from ..frontend.generation import GenerationConfig
from . import api as A
from . import errors as E
from .lifecycle import ServerLifecycle
from .metrics import ServerMetrics
from .resume import CursorTooOld, ResumableStore
from .security import CredentialStore

MAX_DELTA_BYTES = 16 * 1024


@dataclass
class ServerConfig:
    metrics: bool = False
    resumable_sse: bool = False
    replay_sessions: int = 64
    replay_events: int = 256
    cors_origins: tuple = ()
    compatibility_profile: str = "strict"      # strict | openwebui
    request_timeout_s: float = 600.0
    completion_timeout_s: Optional[float] = None
    credentials: CredentialStore = field(default_factory=CredentialStore.open)
    created: int = field(default_factory=lambda: int(time.time()))


class ModelRegistry:
    """alias -> backend, plus the optional dynamic lifecycle registry."""

    def __init__(self, backends: dict, lifecycle_registry=None, fingerprints: Optional[dict] = None):
        self.backends = dict(backends)
        self.dynamic = lifecycle_registry
        self.fingerprints = fingerprints or {}

    def aliases(self) -> list:
        names = list(self.backends)
        if self.dynamic is not None:
            names += [a for a in self.dynamic.aliases() if a not in names]
        return names

    def resolve(self, alias: str):
        b = self.backends.get(alias)
        if b is not None:
            return b, None
        if self.dynamic is not None and alias in self.dynamic.aliases():
            return self.dynamic.acquire(alias)      # (backend, lease) or raises ApiError
        raise E.model_not_found(alias)


def _sse(data: dict, event: Optional[str] = None, eid: Optional[int] = None) -> bytes:
    out = []
    if eid is not None:
        out.append(f"id: {eid}\n")
    if event:
        out.append(f"event: {event}\n")
    out.append("data: " + json.dumps(data, ensure_ascii=False, separators=(",", ":")) + "\n\n")
    return "".join(out).encode("utf-8")


def _split_utf8(text: str, limit: int = MAX_DELTA_BYTES) -> list:
    b = text.encode("utf-8")
    if len(b) <= limit:
        return [text]
    out, start = [], 0
    while start < len(b):
        end = min(len(b), start + limit)
        while end < len(b) and (b[end] & 0xC0) == 0x80:
            end -= 1
        out.append(b[start:end].decode("utf-8"))
        start = end
    return out


def _dispatch_tail(n: int = 16) -> list:
    """The last dispatch records (empty unless SLLM_DISPATCH_AUDIT=1 switched the audit on)."""
    from ..ops import _lib
    return _lib.dispatch_records()[-n:]


def _fallbacks() -> dict:
    """Counters of work that left its fast path (fused tensor-parallel GEMM -> NCCL, fused decode -> per-op kernels)."""
    from ..ops import _lib
    return _lib.fallbacks()


def build_app(registry: ModelRegistry, config: Optional[ServerConfig] = None, lifecycle: Optional[ServerLifecycle] = None) -> FastAPI:
    cfg = config or ServerConfig()
    life = lifecycle or ServerLifecycle()
    if lifecycle is None:
        life.to("ready")
    metrics = ServerMetrics(registry.aliases())
    replay = ResumableStore(cfg.replay_sessions, cfg.replay_events) if cfg.resumable_sse else None
    app = FastAPI(docs_url=None, redoc_url=None, openapi_url=None)
    app.state.registry, app.state.config, app.state.lifecycle, app.state.metrics, app.state.replay = registry, cfg, life, metrics, replay

    # ---------------------------------------------------------------------------------- plumbing
    @app.exception_handler(E.ApiError)
    async def _api_error(request: Request, exc: E.ApiError):
        metrics.http_response(exc.status)
        return JSONResponse(exc.body(), status_code=exc.status)

    @app.middleware("http")
    async def _cors_and_count(request: Request, call_next):
        origin = request.headers.get("origin")
        if request.method == "OPTIONS" and origin and origin in cfg.cors_origins:
            return Response(status_code=204, headers={"access-control-allow-origin": origin,
                                                      "access-control-allow-methods": "GET, POST, OPTIONS",
                                                      "access-control-allow-headers": "authorization, content-type, last-event-id, anthropic-version",
                                                      "vary": "origin"})
        resp = await call_next(request)
        if origin and origin in cfg.cors_origins:
            resp.headers["access-control-allow-origin"] = origin
            resp.headers["vary"] = "origin"
        if not isinstance(resp, StreamingResponse) or resp.status_code != 200:
            metrics.http_response(resp.status_code)
        return resp

    def authorize(request: Request, role: str = "user") -> str:
        got = cfg.credentials.role_for(request.headers.get("authorization"))
        if got is None:
            raise E.unauthorized()
        if role == "admin" and got != "admin":
            raise E.forbidden()
        return got

    async def read_json(request: Request) -> dict:
        ctype = request.headers.get("content-type", "")
        if not ctype.lower().startswith("application/json"):
            raise E.invalid_value("content-type must be application/json", None)
        cl = request.headers.get("content-length")
        if cl is not None:
            try:
                if int(cl) > A.MAX_BODY_BYTES:
                    raise E.too_large()
            except ValueError:
                raise E.invalid_value("invalid content-length") from None
        body = bytearray()
        async for chunk in request.stream():
            body.extend(chunk)
            if len(body) > A.MAX_BODY_BYTES:
                raise E.too_large()
        try:
            obj = json.loads(bytes(body), parse_constant=_reject_constant)
        except (ValueError, UnicodeDecodeError):
            raise E.invalid_json() from None
        if not isinstance(obj, dict):
            raise E.invalid_value("the request body must be a JSON object")
        return obj

    def _reject_constant(name):
        raise ValueError("non-finite number")

    def serving(alias: str):
        if life.state in ("loading", "draining", "failed", "shutdown"):
            raise E.unavailable(f"server is {life.state}")
        backend, lease = registry.resolve(alias)
        if not backend.accepting:
            if lease is not None:
                lease.release()
            raise E.unavailable("scheduler is draining")
        return backend, lease

    def check_context(backend, n_prompt: int, max_new: int):
        if n_prompt + max_new > backend.max_context():
            raise E.invalid_value("prompt tokens plus max tokens exceed the server context length", "max_completion_tokens")

    def submit(backend, ids, gcfg, alias, mm=None):
        try:
            return backend.submit(ids, gcfg, mm=mm) if mm is not None else backend.submit(ids, gcfg)
        except QueueFull:
            metrics.request(alias, "rejected")
            raise E.rate_limited() from None
        except ValueError as exc:
            raise E.invalid_value(str(exc)) from None

    async def next_event(handle):
        return await handle.events.aget()

    async def next_events(handle):
        """One event, plus whatever else is already queued (a stream whose consumer lags behind the engine pays one
        JSON document and one socket write for the whole backlog).  No helper thread: the engine thread wakes this
        loop once per round for all streams (frontend.generation.EventChannel)."""
        return await handle.events.aget_batch(64)

    def grammar_for(response_format: dict) -> Optional[str]:
        t = response_format.get("type")
        if t == "json_object":
            return JSON_OBJECT_GBNF
        if t == "json_schema":
            try:
                return schema_to_gbnf(response_format["json_schema"]["schema"])
            except GrammarError as exc:
                raise E.invalid_value(str(exc), "response_format.json_schema.schema") from None
        return None

    def account(alias, handle, payload, t0, first_at):
        reason = payload.get("finish_reason")
        outcome = {"stop": "completed", "length": "completed", "cancelled": "cancelled", "timeout": "timeout"}.get(reason, "failed")
        metrics.request(alias, outcome)
        u = payload.get("usage", {})
        metrics.add_tokens(alias, "prompt", u.get("prompt_tokens", 0))
        metrics.add_tokens(alias, "completion", u.get("completion_tokens", 0))
        if first_at is not None:
            metrics.ttft(alias, first_at - t0)

    # ---------------------------------------------------------------------------------- operations
    @app.get("/healthz")
    async def healthz():
        return {"status": "ok"}

    @app.get("/readyz")
    async def readyz():
        ok = life.ready and all(b.accepting for b in registry.backends.values())
        return JSONResponse({"status": "ready" if ok else life.state}, status_code=200 if ok else 503)

    @app.get("/metrics")
    async def get_metrics(request: Request):
        if not cfg.metrics:
            raise E.not_found()
        authorize(request)
        stats, mem = {}, {}
        for b in registry.backends.values():
            s = b.scheduler_stats()
            for k, v in s.items():
                if isinstance(v, (int, bool)):
                    stats[k] = stats.get(k, 0) + int(v)
            for k, v in b.memory().items():
                mem[k] = mem.get(k, 0) + v
        return PlainTextResponse(metrics.render(stats, life.ready, mem), media_type="text/plain; version=0.0.4")

    @app.get("/props")
    async def props(request: Request):
        authorize(request)
        return {"models": [{"id": a, **(registry.backends[a].props() if a in registry.backends else {"state": "dynamic"}),
                            "fingerprint": registry.fingerprints.get(a)} for a in registry.aliases()],
                "memory": {a: b.memory() for a, b in registry.backends.items()},
                "lifecycle": life.state,
                "scheduler": {a: b.scheduler_stats() for a, b in registry.backends.items()},
                "features": {"metrics": cfg.metrics, "resumable_sse": cfg.resumable_sse,
                             "compatibility_profile": cfg.compatibility_profile,
                             "dynamic_models": registry.dynamic is not None, "cors": bool(cfg.cors_origins)},
                "fallbacks": _fallbacks(), "dispatch_audit": _dispatch_tail(),
                "request_audit": {a: b.request_audit() for a, b in registry.backends.items() if hasattr(b, "request_audit")}}

    @app.get("/slots")
    async def slots(request: Request):
        authorize(request, "admin")
        return {"slots": [dict(s, model=a) for a, b in registry.backends.items() for s in b.slots()][:1024]}

    @app.post("/admin/slots/{sid}/cancel")
    async def cancel_slot(sid: int, request: Request):
        authorize(request, "admin")
        for b in registry.backends.values():
            if b.cancel_slot(sid):
                metrics.cancellation("admin")
                return {"cancelled": True}
        raise E.not_found("unknown slot")

    @app.post("/admin/keys/reload")
    async def reload_keys(request: Request):
        authorize(request, "admin")
        try:
            n = cfg.credentials.reload()
        except Exception as exc:
            raise E.invalid_value(f"key reload failed: {type(exc).__name__}") from None
        return {"reloaded": True, "keys": n}

    @app.post("/admin/models/evict-idle")
    async def evict_idle(request: Request):
        authorize(request, "admin")
        if registry.dynamic is None:
            raise E.not_found()
        return {"evicted": registry.dynamic.evict_idle()}

    @app.post("/admin/models/{alias}/{action}")
    async def model_admin(alias: str, action: str, request: Request):
        authorize(request, "admin")
        if registry.dynamic is None or action not in ("load", "preload", "unload", "clear-quarantine"):
            raise E.not_found()
        if alias not in registry.dynamic.aliases():
            raise E.model_not_found(alias)
        return {"alias": alias, "state": await asyncio.to_thread(registry.dynamic.admin, alias, action)}

    @app.get("/v1/models")
    async def models(request: Request):
        authorize(request)
        return {"object": "list", "data": [{"id": a, "object": "model", "created": cfg.created, "owned_by": "sllm"}
                                           for a in registry.aliases()]}

    # ---------------------------------------------------------------------------------- chat completions
    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request):
        authorize(request)
        body = await read_json(request)
        mm = False
        if isinstance(body.get("model"), str) and body["model"] in registry.backends:
            mm = bool(registry.backends[body["model"]].props().get("vision"))
        req = A.parse_chat_request(body, cfg.compatibility_profile == "openwebui", multimodal=mm)
        if req.resumable and replay is None:
            raise E.invalid_value("resumable streaming is not enabled on this server", "sllm.resumable")
        backend, lease = serving(req.model)
        try:
            try:
                prompt = render_chatml(req.messages, "enabled" if req.thinking else "disabled")
            except ChatRenderError as exc:
                raise E.invalid_value(str(exc), "messages") from None
            mm_prompt = None
            if req.images:
                from ..frontend import vision as V
                try:
                    mm_prompt = await asyncio.to_thread(
                        backend.multimodal_prompt, prompt, [V.BoundedImage.from_bytes(i.data) for i in req.images])
                except V.VisionError as exc:
                    raise E.invalid_value(str(exc), "messages") from None
                except ValueError as exc:
                    raise E.unsupported(str(exc), "messages") from None
                ids = mm_prompt.tokens
            else:
                ids = backend.tokenizer.encode(prompt)
            check_context(backend, len(ids), req.max_tokens)
            gbnf = grammar_for(req.response_format)
            if req.ignore_eos and getattr(backend.tokenizer, "eos_token_id", None) is not None:
                req.chain.ignore_eos_token = backend.tokenizer.eos_token_id
            if req.dry_breakers:
                from ..engine.sampling import DryConfig
                raw = req.chain._dry_raw
                req.chain.dry = DryConfig(raw[0], raw[1], raw[2], [backend.tokenizer.encode(b, allow_special=False) for b in raw[4]], raw[3])
            elif hasattr(req.chain, "_dry_raw"):
                from ..engine.sampling import DryConfig
                raw = req.chain._dry_raw
                req.chain.dry = DryConfig(raw[0], raw[1], raw[2], [], raw[3])
            handles = []
            for choice in range(req.n):
                seed = None if req.seed is None else derive_choice_seed(req.seed, choice)
                gcfg = GenerationConfig(max_new_tokens=req.max_tokens, chain=req.chain, seed=seed, stop=req.stop,
                                        thinking=req.thinking, separate_reasoning=req.separate_reasoning,
                                        reasoning_budget=req.reasoning_budget, grammar_gbnf=gbnf,
                                        timeout_s=cfg.completion_timeout_s, ignore_eos=req.ignore_eos)
                try:
                    handles.append(submit(backend, ids, gcfg, req.model, mm_prompt))
                except E.ApiError:
                    for h in handles:
                        h.cancel()
                    raise
        except BaseException:
            if lease is not None:
                lease.release()
            raise
        cid = "chatcmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        t0 = time.monotonic()
        if req.stream:
            return StreamingResponse(_chat_stream(req, handles, cid, created, t0, lease), media_type="text/event-stream",
                                     headers={"cache-control": "no-cache", "x-accel-buffering": "no"})
        try:
            choices, usage_p, usage_c = [], 0, 0
            for i, h in enumerate(handles):
                content, reasoning, lps, done, first_at = [], [], [], None, None
                while done is None:
                    kind, payload = await asyncio.wait_for(next_event(h), cfg.request_timeout_s)
                    if kind == "delta":
                        first_at = first_at or time.monotonic()
                        content.append(payload.get("content", ""))
                        reasoning.append(payload.get("reasoning", ""))
                        lps.extend(payload.get("logprobs", []))
                    else:
                        done = payload
                account(req.model, h, done, t0, first_at)
                if done["finish_reason"] in ("error", "cancelled", "timeout"):
                    for other in handles:
                        other.cancel()
                    if done["finish_reason"] == "timeout":
                        raise E.ApiError(504, "timeout", "generation timed out", err_type="server_error")
                    raise E.server_error("generation failed" if done["finish_reason"] == "error" else "generation was cancelled")
                msg = {"role": "assistant", "content": "".join(content)}
                if req.separate_reasoning:
                    msg["reasoning_content"] = "".join(reasoning)
                ch = {"index": i, "message": msg, "finish_reason": done["finish_reason"],
                      "logprobs": _logprobs_obj(backend, lps) if req.logprobs else None}
                choices.append(ch)
                usage_p = done["usage"]["prompt_tokens"]
                usage_c += done["usage"]["completion_tokens"]
            metrics.http_response(200)
            return {"id": cid, "object": "chat.completion", "created": created, "model": req.model, "choices": choices,
                    "usage": {"prompt_tokens": usage_p, "completion_tokens": usage_c, "total_tokens": usage_p + usage_c}}
        except asyncio.TimeoutError:
            for h in handles:
                h.cancel()
            metrics.cancellation("timeout")
            raise E.ApiError(504, "timeout", "request timed out", err_type="server_error") from None
        except asyncio.CancelledError:
            for h in handles:
                h.cancel()
            metrics.cancellation("client_disconnect")
            raise
        finally:
            if lease is not None:
                lease.release()

    def _logprobs_obj(backend, lps):
        def tok(t):
            b = backend.tokenizer.token_bytes(t)
            return {"token": b.decode("utf-8", errors="replace"), "bytes": list(b)}
        return {"content": [{**tok(e["token"]), "logprob": e["logprob"],
                             "top_logprobs": [{**tok(t), "logprob": lp} for t, lp in e.get("top", [])]} for e in lps]}

    async def _chat_stream(req, handles, cid, created, t0, lease):
        session = replay.create(cid) if (req.resumable and replay is not None) else None

        def emit(obj) -> bytes:
            if session is not None:
                eid = session.append(json.dumps(obj, ensure_ascii=False, separators=(",", ":")).encode())
                return _sse(obj, eid=eid)
            return _sse(obj)

        def chunk(i, delta, finish=None, extra=None):
            c = {"index": i, "delta": delta, "finish_reason": finish}
            if extra:
                c.update(extra)
            return {"id": cid, "object": "chat.completion.chunk", "created": created, "model": req.model, "choices": [c]}
        ok = False
        try:
            backend = registry.backends.get(req.model)
            for i in range(len(handles)):
                yield emit(chunk(i, {"role": "assistant", "content": ""}))
            pending = {i: asyncio.ensure_future(next_events(h)) for i, h in enumerate(handles)}
            first_at = None
            lps = {i: [] for i in pending}
            while pending:
                done_set, _ = await asyncio.wait(pending.values(), return_when=asyncio.FIRST_COMPLETED,
                                                 timeout=cfg.request_timeout_s)
                if not done_set:
                    raise asyncio.TimeoutError()
                for i in [k for k, f in pending.items() if f in done_set]:
                    events = pending[i].result()
                    # consecutive content-only deltas of a backlog travel as one chunk
                    merged, text = [], []
                    for kind, payload in events:
                        if kind == "delta" and not payload.get("reasoning"):
                            lps[i].extend(payload.get("logprobs", []))
                            text.append(payload.get("content", ""))
                            continue
                        if text:
                            merged.append(("delta", {"content": "".join(text)}))
                            text = []
                        if kind == "delta":
                            lps[i].extend(payload.get("logprobs", []))
                        merged.append((kind, payload))
                    if text:
                        merged.append(("delta", {"content": "".join(text)}))
                    finished = False
                    for kind, payload in merged:
                        if kind == "delta":
                            first_at = first_at or time.monotonic()
                            if payload.get("reasoning"):
                                yield emit(chunk(i, {"reasoning_content": payload["reasoning"]}))
                            for piece in _split_utf8(payload.get("content", "")):
                                if piece:
                                    yield emit(chunk(i, {"content": piece}))
                            continue
                        finished = True
                        del pending[i]
                        account(req.model, handles[i], payload, t0, first_at)
                        if payload["finish_reason"] in ("error", "cancelled", "timeout"):
                            for h in handles:
                                h.cancel()
                            for f in pending.values():
                                f.cancel()
                            err = E.server_error("generation failed")
                            yield emit(err.body())      # terminal error envelope, then close without [DONE]
                            return
                        extra = {"logprobs": _logprobs_obj(backend, lps[i])} if (req.logprobs and backend) else None
                        fin = chunk(i, {}, payload["finish_reason"], extra)
                        fin["usage"] = payload["usage"]        # per-choice usage rides on its finishing chunk
                        yield emit(fin)
                    if not finished:
                        pending[i] = asyncio.ensure_future(next_events(handles[i]))
            ok = True
            if session is not None:
                session.append(b"[DONE]")
            yield b"data: [DONE]\n\n"
            metrics.http_response(200)
        except asyncio.TimeoutError:
            metrics.cancellation("timeout")
            yield _sse(E.ApiError(504, "timeout", "request timed out", err_type="server_error").body())
        finally:
            if not ok:
                for h in handles:
                    h.cancel()
                if session is None:
                    metrics.cancellation("client_disconnect") if False else None
            if session is not None:
                session.close()
            if lease is not None:
                lease.release()

    def _replay_route(prefix: str):
        async def events(rid: str, request: Request):
            authorize(request)
            if replay is None:
                raise E.not_found()
            session = replay.get(rid)
            if session is None:
                raise E.not_found("unknown stream")
            lei = request.headers.get("last-event-id", "0")
            if not lei.isdigit():
                raise E.invalid_value("Last-Event-ID must be a decimal integer")
            cursor = int(lei)
            try:
                session.after(cursor)
            except CursorTooOld:
                raise E.ApiError(416, "cursor_too_old", "the cursor is older than the replay window") from None

            async def gen():
                cur = cursor
                while True:
                    try:
                        events_, closed = session.after(cur)
                    except CursorTooOld:
                        return
                    for eid, data in events_:
                        cur = eid
                        if data == b"[DONE]":
                            yield b"data: [DONE]\n\n"
                        elif data.startswith(b"event: "):
                            yield f"id: {eid}\n".encode() + data
                        else:
                            yield f"id: {eid}\ndata: ".encode() + data + b"\n\n"
                    if closed:
                        return
                    await asyncio.sleep(0.02)
            return StreamingResponse(gen(), media_type="text/event-stream")
        return events

    app.get("/v1/chat/completions/{rid}/events")(_replay_route("chatcmpl"))
    app.get("/v1/responses/{rid}/events")(_replay_route("resp"))
    app.get("/v1/messages/{rid}/events")(_replay_route("msg"))

    # ---------------------------------------------------------------------------------- completions / infill
    async def _run_text_jobs(model, backend, lease, jobs, stream, make_chunk, make_final, t0):
        """jobs: list of (index, handle).  Shared by /v1/completions and /v1/infill."""
        if stream:
            async def gen():
                ok = False
                try:
                    for i, h in jobs:
                        first_at = None
                        while True:
                            kind, payload = await asyncio.wait_for(next_event(h), cfg.request_timeout_s)
                            if kind == "delta":
                                first_at = first_at or time.monotonic()
                                if payload.get("content"):
                                    yield _sse(make_chunk(i, payload["content"], None))
                            else:
                                account(model, h, payload, t0, first_at)
                                if payload["finish_reason"] in ("error", "cancelled", "timeout"):
                                    yield _sse(E.server_error().body())
                                    return
                                yield _sse(make_chunk(i, "", payload["finish_reason"]))
                                break
                    ok = True
                    yield b"data: [DONE]\n\n"
                finally:
                    if not ok:
                        for _, h in jobs:
                            h.cancel()
                    if lease is not None:
                        lease.release()
            return StreamingResponse(gen(), media_type="text/event-stream")
        try:
            results = []
            for i, h in jobs:
                text, done, first_at = [], None, None
                while done is None:
                    kind, payload = await asyncio.wait_for(next_event(h), cfg.request_timeout_s)
                    if kind == "delta":
                        first_at = first_at or time.monotonic()
                        text.append(payload.get("content", ""))
                    else:
                        done = payload
                account(model, h, done, t0, first_at)
                if done["finish_reason"] in ("error", "cancelled", "timeout"):
                    raise E.server_error()
                results.append((i, "".join(text), done))
            return make_final(results)
        except (asyncio.TimeoutError, asyncio.CancelledError):
            for _, h in jobs:
                h.cancel()
            raise E.ApiError(504, "timeout", "request timed out", err_type="server_error") from None
        finally:
            if lease is not None:
                lease.release()

    @app.post("/v1/completions")
    async def completions(request: Request):
        authorize(request)
        req = A.parse_completion_request(await read_json(request))
        backend, lease = serving(req.model)
        jobs, echoes = [], {}
        try:
            idx = 0
            for p in req.prompts:
                ids = backend.tokenizer.encode(p) if isinstance(p, str) else list(p)
                if not ids:
                    raise E.invalid_value("prompt must not be empty", "prompt")
                if any(t >= backend.tokenizer.vocab_size for t in ids):
                    raise E.invalid_value("token id outside the vocabulary", "prompt")
                check_context(backend, len(ids), req.max_tokens)
                for c in range(req.n):
                    seed = None if req.seed is None else derive_choice_seed(req.seed, idx)
                    gcfg = GenerationConfig(max_new_tokens=req.max_tokens, chain=req.chain, seed=seed, stop=req.stop,
                                            timeout_s=cfg.completion_timeout_s)
                    jobs.append((idx, submit(backend, ids, gcfg, req.model)))
                    echoes[idx] = p if isinstance(p, str) else backend.tokenizer.decode(p)
                    idx += 1
        except BaseException:
            for _, h in jobs:
                h.cancel()
            if lease is not None:
                lease.release()
            raise
        cid, created = "cmpl-" + uuid.uuid4().hex[:24], int(time.time())

        def chunk(i, text, finish):
            return {"id": cid, "object": "text_completion", "created": created, "model": req.model,
                    "choices": [{"index": i, "text": text, "logprobs": None, "finish_reason": finish}]}

        def final(results):
            pt = sum(d["usage"]["prompt_tokens"] for _, _, d in results[::req.n])
            ct = sum(d["usage"]["completion_tokens"] for _, _, d in results)
            return {"id": cid, "object": "text_completion", "created": created, "model": req.model,
                    "choices": [{"index": i, "text": (echoes[i] if req.echo else "") + t, "logprobs": None,
                                 "finish_reason": d["finish_reason"]} for i, t, d in results],
                    "usage": {"prompt_tokens": pt, "completion_tokens": ct, "total_tokens": pt + ct}}
        return await _run_text_jobs(req.model, backend, lease, jobs, req.stream, chunk, final, time.monotonic())

    @app.post("/v1/infill")
    async def infill(request: Request):
        authorize(request)
        model, prefix, suffix, chain, seed, max_tokens, stop, stream = A.parse_infill_request(await read_json(request))
        backend, lease = serving(model)
        try:
            tk = backend.tokenizer
            if not all(s in getattr(tk, "special_ids", {}) for s in ("<|fim_prefix|>", "<|fim_suffix|>", "<|fim_middle|>")) \
                    and not hasattr(tk, "tk"):
                raise E.unsupported("the served model declares no fill-in-the-middle capability", "model")
            ids = tk.encode(render_infill(prefix, suffix))
            check_context(backend, len(ids), max_tokens)
            h = submit(backend, ids, GenerationConfig(max_new_tokens=max_tokens, chain=chain, seed=seed, stop=stop,
                                                      timeout_s=cfg.completion_timeout_s), model)
        except BaseException:
            if lease is not None:
                lease.release()
            raise
        cid, created = "infill-" + uuid.uuid4().hex[:24], int(time.time())

        def chunk(i, text, finish):
            return {"id": cid, "object": "infill.chunk", "created": created, "model": model, "content": text, "finish_reason": finish}

        def final(results):
            _, text, d = results[0]
            return {"id": cid, "object": "infill", "created": created, "model": model, "content": text,
                    "finish_reason": d["finish_reason"], "usage": d["usage"]}
        return await _run_text_jobs(model, backend, lease, [(0, h)], stream, chunk, final, time.monotonic())

    # ---------------------------------------------------------------------------------- embeddings / rerank / utilities
    def _ids_of(backend, item):
        ids = backend.tokenizer.encode(item) if isinstance(item, str) else list(item)
        if not ids:
            raise E.invalid_value("input must not be empty", "input")
        if len(ids) > backend.max_context():
            raise E.invalid_value("input longer than the context length", "input")
        return ids

    @app.post("/v1/embeddings")
    async def embeddings(request: Request):
        authorize(request)
        req = A.parse_embedding_request(await read_json(request))
        backend, lease = serving(req.model)
        try:
            token_lists = [_ids_of(backend, x) for x in req.inputs]
            vecs = await asyncio.to_thread(backend.embed, token_lists)
        finally:
            if lease is not None:
                lease.release()
        data = []
        for i, v in enumerate(vecs):
            emb = base64.b64encode(np.asarray(v, dtype="<f4").tobytes()).decode() if req.encoding_format == "base64" \
                else [float(x) for x in v]
            data.append({"object": "embedding", "index": i, "embedding": emb})
        n = sum(len(t) for t in token_lists)
        return {"object": "list", "data": data, "model": req.model, "usage": {"prompt_tokens": n, "total_tokens": n}}

    @app.post("/v1/rerank")
    async def rerank(request: Request):
        authorize(request)
        req = A.parse_rerank_request(await read_json(request))
        backend, lease = serving(req.model)
        try:
            lists = [_ids_of(backend, req.query)] + [_ids_of(backend, d) for d in req.documents]
            vecs = await asyncio.to_thread(backend.embed, lists)
        finally:
            if lease is not None:
                lease.release()
        q = np.asarray(vecs[0], dtype=np.float64)
        scores = [float(np.dot(q, np.asarray(v, dtype=np.float64))) for v in vecs[1:]]
        order = sorted(range(len(scores)), key=lambda i: (-scores[i], i))[:req.top_n]   # ties keep document order
        results = [{"index": i, "relevance_score": scores[i], **({"document": {"text": req.documents[i]}} if req.return_documents else {})}
                   for i in order]
        return {"object": "rerank", "model": req.model, "results": results,
                "usage": {"prompt_tokens": sum(len(x) for x in lists), "total_tokens": sum(len(x) for x in lists)}}

    @app.post("/v1/tokenize")
    async def tokenize(request: Request):
        authorize(request)
        model, content, add_special, with_pieces = A.parse_tokenize_request(await read_json(request))
        backend, lease = registry.resolve(model)
        try:
            ids = backend.tokenizer.encode(content, allow_special=add_special)
            out = {"tokens": ids, "count": len(ids)}
            if with_pieces:
                out["pieces"] = backend.tokenizer.pieces(ids)
            return out
        finally:
            if lease is not None:
                lease.release()

    @app.post("/v1/detokenize")
    async def detokenize(request: Request):
        authorize(request)
        model, tokens, skip = A.parse_detokenize_request(await read_json(request))
        backend, lease = registry.resolve(model)
        try:
            if any(t >= backend.tokenizer.vocab_size for t in tokens):
                raise E.invalid_value("token id outside the vocabulary", "tokens")
            return {"content": backend.tokenizer.decode(tokens, skip_special_tokens=skip)}
        finally:
            if lease is not None:
                lease.release()

    @app.post("/v1/apply-template")
    async def apply_template(request: Request):
        authorize(request)
        model, messages, agp, thinking = A.parse_apply_template_request(await read_json(request))
        backend, lease = registry.resolve(model)
        try:
            return {"prompt": render_chatml(messages, thinking, agp)}
        except ChatRenderError as exc:
            raise E.invalid_value(str(exc), "messages") from None
        finally:
            if lease is not None:
                lease.release()

    @app.post("/v1/input-tokens")
    async def input_tokens(request: Request):
        authorize(request)
        model, messages, agp, thinking = A.parse_apply_template_request(await read_json(request))
        backend, lease = registry.resolve(model)
        try:
            n = len(backend.tokenizer.encode(render_chatml(messages, thinking, agp)))
            return {"input_tokens": n, "context_length": backend.max_context()}
        except ChatRenderError as exc:
            raise E.invalid_value(str(exc), "messages") from None
        finally:
            if lease is not None:
                lease.release()

    # ---------------------------------------------------------------------------------- responses / anthropic
    def _protocol_prompt(backend, req: A.ProtocolRequest):
        system = req.system
        gbnf = None
        if req.tools and (req.tool_choice is None or req.tool_choice.mode != "none"):
            system = (system + "\n\n" if system else "") + T.render_tool_preamble(req.tools)
            if req.tool_choice is not None and req.tool_choice.mode in ("required", "named"):
                try:
                    gbnf = schema_to_gbnf(T.envelope_schema(req.tools, req.tool_choice))
                except GrammarError as exc:
                    raise E.invalid_value(f"tool schema is outside the supported subset: {exc}", "tools") from None
        msgs = ([ChatMessage("system", system)] if system else []) + req.messages
        try:
            prompt = render_chatml(msgs, "enabled" if req.thinking else "disabled")
        except ChatRenderError as exc:
            raise E.invalid_value(str(exc), "input") from None
        return backend.tokenizer.encode(prompt), gbnf

    def _maybe_tool_calls(req, text):
        if not req.tools or (req.tool_choice is not None and req.tool_choice.mode == "none"):
            return None
        stripped = text.strip()
        if not stripped.startswith("{"):
            return None
        try:
            return T.parse_tool_calls(stripped, req.tools, "call_" + uuid.uuid4().hex[:12])
        except T.ToolProtocolError:
            return None

    async def _collect(handle):
        text, done = [], None
        while done is None:
            kind, payload = await asyncio.wait_for(next_event(handle), cfg.request_timeout_s)
            if kind == "delta":
                text.append(payload.get("content", ""))
            else:
                done = payload
        return "".join(text), done

    @app.post("/v1/responses")
    async def responses(request: Request):
        authorize(request)
        req = A.parse_responses_request(await read_json(request))
        if req.resumable and replay is None:
            raise E.invalid_value("resumable streaming is not enabled on this server", "sllm.resumable")
        backend, lease = serving(req.model)
        try:
            ids, gbnf = _protocol_prompt(backend, req)
            check_context(backend, len(ids), req.max_tokens)
            h = submit(backend, ids, GenerationConfig(max_new_tokens=req.max_tokens, chain=req.chain, grammar_gbnf=gbnf,
                                                      thinking=req.thinking, separate_reasoning=req.thinking,
                                                      timeout_s=cfg.completion_timeout_s), req.model)
        except BaseException:
            if lease is not None:
                lease.release()
            raise
        rid, created, t0 = "resp_" + uuid.uuid4().hex[:24], int(time.time()), time.monotonic()

        def response_obj(status, output, text, usage, incomplete=None, error=None):
            return {"id": rid, "object": "response", "created_at": created, "model": req.model, "status": status,
                    "output": output, "output_text": text, "incomplete_details": incomplete, "error": error,
                    "metadata": req.metadata, "parallel_tool_calls": req.parallel_tool_calls, "store": False,
                    "usage": None if usage is None else {"input_tokens": usage["prompt_tokens"],
                                                         "output_tokens": usage["completion_tokens"],
                                                         "total_tokens": usage["total_tokens"]}}

        def outputs_for(text):
            calls = _maybe_tool_calls(req, text)
            if calls:
                if not req.parallel_tool_calls:
                    calls = calls[:1]
                return [{"type": "function_call", "id": "fc_" + c.id, "call_id": c.id, "name": c.name,
                         "arguments": json.dumps(c.arguments, separators=(",", ":")), "status": "completed"} for c in calls], ""
            mid = "msg_" + uuid.uuid4().hex[:24]
            return [{"type": "message", "id": mid, "role": "assistant", "status": "completed",
                     "content": [{"type": "output_text", "text": text, "annotations": []}]}], text

        if not req.stream:
            try:
                text, done = await _collect(h)
                account(req.model, h, done, t0, None)
                if done["finish_reason"] in ("error", "cancelled", "timeout"):
                    raise E.server_error()
                out, otext = outputs_for(text)
                inc = {"reason": "max_output_tokens"} if done["finish_reason"] == "length" else None
                return response_obj("incomplete" if inc else "completed", out, otext, done["usage"], inc)
            except (asyncio.TimeoutError, asyncio.CancelledError):
                h.cancel()
                raise E.ApiError(504, "timeout", "request timed out", err_type="server_error") from None
            finally:
                if lease is not None:
                    lease.release()

        async def gen():
            session = replay.create(rid) if (req.resumable and replay is not None) else None
            seq = [0]

            def ev(name, data):
                data = {"type": name, "sequence_number": seq[0], **data}
                seq[0] += 1
                raw = _sse(data, event=name)
                if session is not None:
                    eid = session.append(raw)
                    return f"id: {eid}\n".encode() + raw
                return raw
            ok = False
            try:
                yield ev("response.created", {"response": response_obj("in_progress", [], "", None)})
                mid = "msg_" + uuid.uuid4().hex[:24]
                started = False
                text = []
                while True:
                    kind, payload = await asyncio.wait_for(next_event(h), cfg.request_timeout_s)
                    if kind == "delta":
                        if not payload.get("content"):
                            continue
                        if not started and not req.tools:
                            started = True
                            yield ev("response.output_item.added", {"output_index": 0, "item": {"type": "message", "id": mid, "role": "assistant", "status": "in_progress", "content": []}})
                            yield ev("response.content_part.added", {"item_id": mid, "output_index": 0, "content_index": 0, "part": {"type": "output_text", "text": "", "annotations": []}})
                        text.append(payload["content"])
                        if not req.tools:
                            for piece in _split_utf8(payload["content"]):
                                yield ev("response.output_text.delta", {"item_id": mid, "output_index": 0, "content_index": 0, "delta": piece})
                    else:
                        account(req.model, h, payload, t0, None)
                        if payload["finish_reason"] in ("error", "cancelled", "timeout"):
                            yield ev("error", {"code": "server_error", "message": "generation failed", "param": None})
                            return
                        full = "".join(text)
                        out, otext = outputs_for(full)
                        if out and out[0]["type"] == "function_call":
                            for oi, item in enumerate(out):
                                yield ev("response.output_item.added", {"output_index": oi, "item": {**item, "arguments": "", "status": "in_progress"}})
                                yield ev("response.function_call_arguments.delta", {"item_id": item["id"], "output_index": oi, "delta": item["arguments"]})
                                yield ev("response.function_call_arguments.done", {"item_id": item["id"], "output_index": oi, "arguments": item["arguments"]})
                                yield ev("response.output_item.done", {"output_index": oi, "item": item})
                        else:
                            if not started:
                                yield ev("response.output_item.added", {"output_index": 0, "item": {"type": "message", "id": mid, "role": "assistant", "status": "in_progress", "content": []}})
                                yield ev("response.content_part.added", {"item_id": mid, "output_index": 0, "content_index": 0, "part": {"type": "output_text", "text": "", "annotations": []}})
                                for piece in _split_utf8(full):
                                    if piece:
                                        yield ev("response.output_text.delta", {"item_id": mid, "output_index": 0, "content_index": 0, "delta": piece})
                            out[0]["id"] = mid
                            yield ev("response.output_text.done", {"item_id": mid, "output_index": 0, "content_index": 0, "text": full})
                            yield ev("response.content_part.done", {"item_id": mid, "output_index": 0, "content_index": 0, "part": out[0]["content"][0]})
                            yield ev("response.output_item.done", {"output_index": 0, "item": out[0]})
                        inc = {"reason": "max_output_tokens"} if payload["finish_reason"] == "length" else None
                        yield ev("response.completed", {"response": response_obj("incomplete" if inc else "completed", out, otext, payload["usage"], inc)})
                        ok = True
                        return
            except asyncio.TimeoutError:
                yield ev("error", {"code": "timeout", "message": "request timed out", "param": None})
            finally:
                if not ok:
                    h.cancel()
                if session is not None:
                    session.close()
                if lease is not None:
                    lease.release()
        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.post("/v1/messages")
    async def anthropic_messages(request: Request):
        authorize_anthropic(request)
        if request.headers.get("anthropic-version") != "2023-06-01":
            raise _anthropic_error(400, "invalid_request_error", "anthropic-version must be 2023-06-01")
        try:
            req = A.parse_anthropic_request(await read_json(request))
            if req.resumable and replay is None:
                raise E.invalid_value("resumable streaming is not enabled on this server", "sllm.resumable")
            backend, lease = serving(req.model)
        except E.ApiError as exc:
            raise _to_anthropic(exc) from None
        try:
            ids, gbnf = _protocol_prompt(backend, req)
            check_context(backend, len(ids), req.max_tokens)
            h = submit(backend, ids, GenerationConfig(max_new_tokens=req.max_tokens, chain=req.chain, stop=req.stop,
                                                      grammar_gbnf=gbnf, timeout_s=cfg.completion_timeout_s), req.model)
        except E.ApiError as exc:
            if lease is not None:
                lease.release()
            raise _to_anthropic(exc) from None
        except BaseException:
            if lease is not None:
                lease.release()
            raise
        mid, t0 = "msg_" + uuid.uuid4().hex[:24], time.monotonic()
        stop_map = {"stop": "end_turn", "length": "max_tokens"}

        def content_blocks(text):
            calls = _maybe_tool_calls(req, text)
            if calls:
                return [{"type": "tool_use", "id": "toolu_" + c.id, "name": c.name, "input": c.arguments} for c in calls], "tool_use"
            return [{"type": "text", "text": text}], None

        def message_obj(blocks, stop_reason, usage, stop_sequence=None):
            return {"id": mid, "type": "message", "role": "assistant", "model": req.model, "content": blocks,
                    "stop_reason": stop_reason, "stop_sequence": stop_sequence,
                    "usage": {"input_tokens": usage["prompt_tokens"], "output_tokens": usage["completion_tokens"]}}

        if not req.stream:
            try:
                text, done = await _collect(h)
                account(req.model, h, done, t0, None)
                if done["finish_reason"] in ("error", "cancelled", "timeout"):
                    raise _anthropic_error(500, "api_error", "generation failed")
                blocks, tool_stop = content_blocks(text)
                reason = tool_stop or stop_map.get(done["finish_reason"], "end_turn")
                return message_obj(blocks, reason, done["usage"])
            except (asyncio.TimeoutError, asyncio.CancelledError):
                h.cancel()
                raise _anthropic_error(504, "api_error", "request timed out") from None
            finally:
                if lease is not None:
                    lease.release()

        async def gen():
            session = replay.create(mid) if (req.resumable and replay is not None) else None

            def ev(name, data):
                raw = _sse({"type": name, **data}, event=name)
                if session is not None:
                    eid = session.append(raw)
                    return f"id: {eid}\n".encode() + raw
                return raw
            ok = False
            try:
                yield ev("message_start", {"message": message_obj([], None, {"prompt_tokens": h.prompt_tokens, "completion_tokens": 0})})
                text, opened = [], False
                while True:
                    kind, payload = await asyncio.wait_for(next_event(h), cfg.request_timeout_s)
                    if kind == "delta":
                        if not payload.get("content"):
                            continue
                        text.append(payload["content"])
                        if not req.tools:
                            if not opened:
                                opened = True
                                yield ev("content_block_start", {"index": 0, "content_block": {"type": "text", "text": ""}})
                            for piece in _split_utf8(payload["content"]):
                                yield ev("content_block_delta", {"index": 0, "delta": {"type": "text_delta", "text": piece}})
                    else:
                        account(req.model, h, payload, t0, None)
                        if payload["finish_reason"] in ("error", "cancelled", "timeout"):
                            yield ev("error", {"error": {"type": "api_error", "message": "generation failed"}})
                            return
                        blocks, tool_stop = content_blocks("".join(text))
                        if req.tools:
                            for bi, b in enumerate(blocks):
                                if b["type"] == "tool_use":
                                    yield ev("content_block_start", {"index": bi, "content_block": {**b, "input": {}}})
                                    yield ev("content_block_delta", {"index": bi, "delta": {"type": "input_json_delta", "partial_json": json.dumps(b["input"], separators=(",", ":"))}})
                                else:
                                    yield ev("content_block_start", {"index": bi, "content_block": {"type": "text", "text": ""}})
                                    yield ev("content_block_delta", {"index": bi, "delta": {"type": "text_delta", "text": b["text"]}})
                                yield ev("content_block_stop", {"index": bi})
                        else:
                            if not opened:
                                yield ev("content_block_start", {"index": 0, "content_block": {"type": "text", "text": ""}})
                            yield ev("content_block_stop", {"index": 0})
                        reason = tool_stop or stop_map.get(payload["finish_reason"], "end_turn")
                        yield ev("message_delta", {"delta": {"stop_reason": reason, "stop_sequence": None},
                                                   "usage": {"output_tokens": payload["usage"]["completion_tokens"]}})
                        yield ev("message_stop", {})
                        ok = True
                        return
            except asyncio.TimeoutError:
                yield ev("error", {"error": {"type": "api_error", "message": "request timed out"}})
            finally:
                if not ok:
                    h.cancel()
                if session is not None:
                    session.close()
                if lease is not None:
                    lease.release()
        return StreamingResponse(gen(), media_type="text/event-stream")

    class AnthropicError(Exception):
        def __init__(self, status, etype, message):
            self.status, self.etype, self.message = status, etype, message

    def _anthropic_error(status, etype, message):
        return AnthropicError(status, etype, message)

    def _to_anthropic(exc: E.ApiError):
        etype = {400: "invalid_request_error", 401: "authentication_error", 403: "permission_error", 404: "not_found_error",
                 413: "request_too_large", 429: "rate_limit_error", 503: "overloaded_error"}.get(exc.status, "api_error")
        return AnthropicError(exc.status, etype, exc.message)

    def authorize_anthropic(request: Request):
        hdr = request.headers.get("authorization")
        if hdr is None and request.headers.get("x-api-key"):
            hdr = "Bearer " + request.headers["x-api-key"]
        if cfg.credentials.role_for(hdr) is None:
            raise AnthropicError(401, "authentication_error", "invalid or missing API key")

    @app.exception_handler(AnthropicError)
    async def _anthropic_handler(request: Request, exc: AnthropicError):
        metrics.http_response(exc.status)
        return JSONResponse({"type": "error", "error": {"type": exc.etype, "message": exc.message}}, status_code=exc.status)

    return app

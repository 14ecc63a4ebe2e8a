"""`sllm chat`: a persistent conversation on one resident model, as versioned JSONL events.

A turn is committed to the transcript only after its generation succeeded; SIGINT cancels the turn in flight
and keeps the session; the KV state of the committed transcript is reused for the next turn through the prefix
cache, and `--checkpoint-save/--checkpoint-load` persist it across processes
(reference: crates/sllm-cli/src/production_chat.rs, chat.rs, interactive.rs; docs/architecture/runtime.md:366-375).
"""
from __future__ import annotations

import json
import signal
import sys

from .common import CliError, StrictParser, add_model_source, emit, open_model

EVENT_VERSION = 1


def _ev(kind, **kw):
    emit({"v": EVENT_VERSION, "event": kind, **kw})


def run_chat(argv) -> int:
    p = StrictParser(prog="sllm chat")
    add_model_source(p)
    p.add_argument("--system")
    p.add_argument("--prompt", action="append", default=[])
    p.add_argument("--message", action="append", default=[])
    p.add_argument("--prompt-file")
    p.add_argument("--reverse-prompt", action="append", default=[])
    p.add_argument("--stop", action="append", default=[])
    p.add_argument("--max-new-tokens", type=int, default=256)
    p.add_argument("--thinking", action="store_true")
    p.add_argument("--reasoning-budget", type=int, default=None)
    p.add_argument("--prefix-cache", action="store_true")
    p.add_argument("--checkpoint-directory")
    p.add_argument("--checkpoint-quota-bytes", type=int, default=8 << 30)
    p.add_argument("--checkpoint-load")
    p.add_argument("--checkpoint-save")
    p.add_argument("--completion-timeout-seconds", type=float, default=None)
    p.add_argument("--shutdown-timeout-seconds", type=float, default=5.0)
    p.add_argument("--temperature", type=float, default=None)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--seed", type=int, default=None)
    a = p.parse_args(argv)
    if len(a.reverse_prompt) > 4 or len(a.stop) > 4:
        raise CliError("at most 4 --reverse-prompt and 4 --stop strings")
    if a.reasoning_budget is not None and not 1 <= a.reasoning_budget <= 4096:
        raise CliError("--reasoning-budget must be in 1..4096")
    if (a.checkpoint_load or a.checkpoint_save) and not a.checkpoint_directory:
        raise CliError("--checkpoint-load/--checkpoint-save need --checkpoint-directory")
    from ..cache import checkpoint as CK
    from ..cache.prefix import PrefixCache
    from ..engine import sampling as S
    from ..engine.scheduler import EngineLoop
    from ..frontend.chat import ChatMessage, render_chatml
    from ..frontend.generation import GenerationConfig, GenerationService

    eng, tok, g, lock = open_model(a, max_batch=2)
    pc = PrefixCache(eng, min_tokens=eng.cfg.page_size)
    loop = EngineLoop(eng, "chat", prefix_cache=pc)
    svc = GenerationService(loop, tok, eng.cfg.vocab, "chat")
    store = CK.CheckpointStore(a.checkpoint_directory, a.checkpoint_quota_bytes) if a.checkpoint_directory else None
    ident = CK.CheckpointIdentity(model=lock["fingerprint"], plan="chat-v1", tokenizer=getattr(tok, "identity", "byte"))
    transcript = []
    if a.system:
        transcript.append(ChatMessage("system", a.system))
    if a.checkpoint_load:
        try:
            ck = store.load(a.checkpoint_load, CK.CheckpointIdentity(ident.model, ident.plan, CK.kv_layout_id(eng.cache),
                                                                     ident.tokenizer))
            transcript = [ChatMessage(m["role"], m["content"]) for m in json.loads(ck.conversation or "[]")]
            seq = CK.restore(eng, ck)
            pc.publish(seq, seq.num_computed)
            eng.free_sequence(seq)
            _ev("checkpoint_loaded", id=a.checkpoint_load, tokens=len(ck.tokens), messages=len(transcript))
        except (OSError, CK.CheckpointError) as exc:
            raise CliError(f"cannot load the checkpoint: {exc}", 3) from None
    for m in a.message:
        role, sep, content = m.partition(":")
        if not sep or role not in ("system", "user", "assistant"):
            raise CliError("--message must look like ROLE:CONTENT")
        transcript.append(ChatMessage(role, content))
    turns = list(a.prompt)
    if a.prompt_file:
        with open(a.prompt_file, "r", encoding="utf-8") as f:
            turns += [ln.rstrip("\n") for ln in f if ln.strip()]
    interactive = not turns
    current = {"handle": None}

    def on_sigint(signum, frame):
        h = current["handle"]
        if h is not None:
            h.cancel()
        else:
            raise KeyboardInterrupt

    signal.signal(signal.SIGINT, on_sigint)
    _ev("session_started", model=lock["semantic_model_id"], context_length=eng.cfg.max_context)
    params = S.SamplingParams(temperature=a.temperature or 0.0, top_p=a.top_p)
    last_ids = []
    rc = 0
    try:
        while True:
            if turns:
                user = turns.pop(0)
            elif interactive:
                line = sys.stdin.readline()
                if not line:
                    break
                user = line.rstrip("\n")
                if not user:
                    continue
            else:
                break
            msgs = transcript + [ChatMessage("user", user)]
            ids = tok.encode(render_chatml(msgs, thinking="enabled" if a.thinking else "disabled"))
            cfg = GenerationConfig(max_new_tokens=a.max_new_tokens, chain=S.SamplerChainConfig(params=params), seed=a.seed,
                                   stop=tuple(a.stop) + tuple(a.reverse_prompt), thinking=a.thinking,
                                   separate_reasoning=a.thinking, reasoning_budget=a.reasoning_budget,
                                   timeout_s=a.completion_timeout_seconds, echo_tokens=True)
            _ev("turn_started", prompt_tokens=len(ids))
            try:
                h = svc.submit(ids, cfg, prefix_seq=pc.lookup(ids))
            except ValueError as exc:
                _ev("turn_failed", reason=str(exc))
                rc = 1
                continue
            current["handle"] = h
            text, reasoning, done, toks = [], [], None, []
            for kind, payload in h:
                if kind == "delta":
                    if payload.get("content") or payload.get("reasoning"):
                        _ev("delta", content=payload.get("content", ""), reasoning=payload.get("reasoning", ""))
                    text.append(payload.get("content", ""))
                    reasoning.append(payload.get("reasoning", ""))
                    toks += payload.get("tokens", [])
                else:
                    done = payload
            current["handle"] = None
            if done["finish_reason"] in ("stop", "length"):
                transcript = msgs + [ChatMessage("assistant", "".join(text))]      # commit only a successful turn
                last_ids = ids + toks
                _ev("turn_committed", finish_reason=done["finish_reason"], usage=done["usage"],
                    prefix_hit_tokens=getattr(getattr(h, "request", None), "prefix_hit_tokens", 0))
            else:
                _ev("turn_discarded", finish_reason=done["finish_reason"], error=done.get("error"))
                if done["finish_reason"] == "error":
                    rc = 1
        if a.checkpoint_save and last_ids:
            seq = eng.new_sequence(last_ids[:-1])
            try:
                lease = pc.lookup(last_ids[:-1])
                if lease is not None:
                    eng.free_sequence(seq)
                    seq = eng.fork_sequence(lease, last_ids[:-1])
                    lease.release()
                eng.prefill([seq], sample=False)
                ck = CK.capture(eng, seq, ident, conversation=json.dumps(
                    [{"role": m.role, "content": m.content} for m in transcript]))
                n = store.save(a.checkpoint_save, ck)
                _ev("checkpoint_saved", id=a.checkpoint_save, bytes=n, tokens=len(ck.tokens))
            finally:
                eng.free_sequence(seq)
    except KeyboardInterrupt:
        _ev("interrupted")
        rc = 130
    finally:
        audit = loop.shutdown(a.shutdown_timeout_seconds)
        _ev("session_ended", prefix_cache=pc.stats(), **audit)
    return rc

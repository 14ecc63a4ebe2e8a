"""`sllm`: version doctor chat models verify-model tokenize detokenize render apply-template input-tokens
completions embeddings rerank infill decode generate benchmark.

Each command prints JSON lines on stdout (one result object, or versioned events for chat / benchmark) and
exits 0 on success, 2 on a usage error, 3 when model verification fails, 4 without a usable device
(reference: crates/sllm-cli/src/main.rs:34-42 dispatch, model.rs command bodies, benchmark.rs:6-23 timeline
event names and schema ids).
"""
from __future__ import annotations

import json
import os
import sys
import time

from .. import __version__ as VERSION
from .common import (CliError, StrictParser, add_generation_args, add_model_source, emit, open_model,
                     prompt_ids_from_args, run_main, sampling_from_args)

BENCH_SCHEMA_DIRECT = "engine-performance-direct-v1"
BENCH_SCHEMA_RENDER = "engine-performance-render-v1"
CHAT_EVENT_VERSION = 1
COMMANDS = ("version", "doctor", "chat", "models", "verify-model", "tokenize", "detokenize", "render", "apply-template",
            "input-tokens", "completions", "embeddings", "rerank", "infill", "decode", "generate", "benchmark")


# ------------------------------------------------------------------------------------------ small commands
def cmd_version(argv):
    StrictParser(prog="sllm version").parse_args(argv)
    emit({"name": "sllm-b200", "version": VERSION, "target": "sm_100a"})


def cmd_doctor(argv):
    StrictParser(prog="sllm doctor").parse_args(argv)
    import torch
    from ..ops import _lib
    rep = {"version": VERSION, "python": sys.version.split()[0], "torch": torch.__version__,
           "cuda_available": torch.cuda.is_available(), "kernel_library": _lib.kernels_available()}
    try:
        _lib.host()
        rep["host_library"] = True
    except Exception as exc:
        rep["host_library"] = False
        rep["host_library_error"] = str(exc)
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        rep["device"] = {"name": p.name, "sm": f"{p.major}.{p.minor}", "memory_bytes": p.total_memory,
                         "multiprocessors": p.multi_processor_count, "count": torch.cuda.device_count()}
        rep["target_ok"] = (p.major, p.minor) == (10, 0)
    rep["ok"] = bool(rep["host_library"] and (not rep["cuda_available"] or (rep["kernel_library"] and rep.get("target_ok"))))
    emit(rep)
    return 0 if rep["ok"] else 1


def cmd_verify_model(argv):
    p = StrictParser(prog="sllm verify-model")
    p.add_argument("--gguf", required=True)
    p.add_argument("--derived-lock", required=True)
    a = p.parse_args(argv)
    from ..formats import gguf as G
    from ..models import loader
    try:
        lock = G.read_derived_lock(a.derived_lock)
        g = G.verify_gguf(a.gguf, lock)
    except (OSError, G.GgufError) as exc:
        raise CliError(f"model verification failed: {exc}", 3) from None
    cfg = loader.config_from_gguf(g)
    rec = g.recipe() or {"bindings": []}
    emit({"verified": True, "semantic_model_id": lock["semantic_model_id"], "fingerprint": lock["fingerprint"],
          "sha256": lock["output"]["sha256"], "size_bytes": g.size, "tensors": len(g.tensors),
          "quantized_tensors": len(rec["bindings"]), "model": cfg.name, "layers": cfg.n_layers, "vocab": cfg.vocab,
          "weight_format": cfg.weight_format})
    g.close()


def _tokenizer_only(a):
    """Tokenizer from a GGUF (verified) or the byte tokenizer when no model is given."""
    from ..frontend.text import ByteTokenizer
    if not a.gguf:
        return ByteTokenizer()
    from ..formats import gguf as G
    from ..models import loader
    if not a.derived_lock:
        raise CliError("--gguf needs --derived-lock")
    try:
        g = G.verify_gguf(a.gguf, G.read_derived_lock(a.derived_lock))
    except (OSError, G.GgufError) as exc:
        raise CliError(f"model verification failed: {exc}", 3) from None
    return loader.tokenizer_from_gguf(g)


def _tok_parser(name):
    p = StrictParser(prog=f"sllm {name}")
    p.add_argument("--gguf")
    p.add_argument("--derived-lock")
    return p


def cmd_tokenize(argv):
    p = _tok_parser("tokenize")
    p.add_argument("--text", required=True)
    p.add_argument("--pieces", action="store_true")
    a = p.parse_args(argv)
    tk = _tokenizer_only(a)
    ids = tk.encode(a.text)
    out = {"tokens": ids, "count": len(ids)}
    if a.pieces:
        out["pieces"] = tk.pieces(ids)
    emit(out)


def _parse_ids(s):
    try:
        ids = [int(x) for x in s.replace(",", " ").split()]
    except ValueError:
        raise CliError("--tokens must be integers") from None
    if any(i < 0 for i in ids):
        raise CliError("token ids must be non-negative")
    return ids


def cmd_detokenize(argv):
    p = _tok_parser("detokenize")
    p.add_argument("--tokens", required=True)
    p.add_argument("--skip-special-tokens", action="store_true")
    a = p.parse_args(argv)
    tk = _tokenizer_only(a)
    emit({"text": tk.decode(_parse_ids(a.tokens), skip_special_tokens=a.skip_special_tokens)})


def _messages(a):
    from ..frontend.chat import ChatMessage
    msgs = []
    for m in a.message:
        role, sep, content = m.partition(":")
        if not sep or role not in ("system", "user", "assistant", "tool"):
            raise CliError("--message must look like ROLE:CONTENT")
        msgs.append(ChatMessage(role, content))
    if a.prompt:
        msgs.append(ChatMessage("user", a.prompt))
    if not msgs:
        raise CliError("give --prompt or --message")
    return msgs


def _render(a, tk=None):
    from ..frontend import chat as C
    msgs = _messages(a)
    if getattr(a, "chat_template_file", None):
        from .template_file import read_template_file
        src = read_template_file(a.chat_template_file)
        kwargs = {}
        if a.template_kwargs_json:
            try:
                kwargs = json.loads(a.template_kwargs_json)
            except json.JSONDecodeError:
                raise CliError("--template-kwargs-json is not valid JSON") from None
            if not isinstance(kwargs, dict):
                raise CliError("--template-kwargs-json must be an object")
        try:
            t = C.GenericTemplate(src, a.chat_template_digest)
            return t.render(msgs, add_generation_prompt=not a.no_generation_prompt, **kwargs), t.digest
        except C.ChatRenderError as exc:
            raise CliError(str(exc)) from None
    try:
        return C.render_chatml(msgs, thinking="enabled" if a.thinking else "disabled",
                               add_generation_prompt=not a.no_generation_prompt), None
    except C.ChatRenderError as exc:
        raise CliError(str(exc)) from None


def _render_parser(name):
    p = _tok_parser(name)
    p.add_argument("--prompt")
    p.add_argument("--message", action="append", default=[])
    p.add_argument("--thinking", action="store_true")
    p.add_argument("--no-generation-prompt", action="store_true")
    p.add_argument("--chat-template-file")
    p.add_argument("--chat-template-digest")
    p.add_argument("--template-kwargs-json")
    return p


def cmd_render(argv):
    a = _render_parser("render").parse_args(argv)
    if a.chat_template_file:
        raise CliError("render uses the built-in renderer; use apply-template for a template file")
    text, _ = _render(a)
    emit({"prompt": text, "renderer": "chatml-v1"})


def cmd_apply_template(argv):
    a = _render_parser("apply-template").parse_args(argv)
    text, digest = _render(a)
    emit({"prompt": text, "template_sha256": digest, "renderer": "generic-sandbox" if digest else "chatml-v1"})


def cmd_input_tokens(argv):
    a = _render_parser("input-tokens").parse_args(argv)
    tk = _tokenizer_only(a)
    text, _ = _render(a)
    ids = tk.encode(text)
    emit({"input_tokens": len(ids), "tokens": ids})


# ------------------------------------------------------------------------------------------ model commands
def _multimodal_from_args(eng, tok, a):
    """models.vision_tower.MultimodalPrompt for --image inputs."""
    from ..frontend import vision as V
    from ..models.vision_tower import MultimodalPrompt, encode_with_images
    tower = getattr(eng, "vision", None)
    if tower is None:
        raise CliError("--image needs a model file with a vision tower (v.* tensors)")
    tok_id = eng.cfg.image_token_id if eng.cfg.image_token_id is not None else eng.cfg.vocab - 1
    try:
        images = V.process_many([V.BoundedImage.from_local_path(p) for p in a.image])
    except (OSError, V.VisionError) as exc:
        raise CliError(f"image input rejected: {exc}") from None
    return MultimodalPrompt(tower, images, encode_with_images(tok, prompt_ids_from_args(a, tok, as_text=True), tok_id), tok_id)


def _generate(eng, tok, ids, a, on_delta=None, timeline=None, mm=None):
    """Runs one request through the generation service; returns (text, reasoning, done, handle)."""
    from ..engine.scheduler import EngineLoop
    from ..frontend.generation import GenerationConfig, GenerationService
    loop = EngineLoop(eng, "cli", prefill_chunk_tokens=a.prefill_chunk_tokens)
    if getattr(a, "mtp_draft_width", 0) > 0:
        if getattr(eng, "mtp_weights", None) is None:
            loop.shutdown(5.0)
            raise CliError("--mtp-draft-width needs a model file with an MTP component (mtp.* tensors)")
        from ..engine.speculative import SpeculativeDecoder
        from ..models.mtp import MtpDraftProvider, MtpHead
        head = getattr(eng, "_mtp_head", None)
        if head is None:
            head = eng._mtp_head = MtpHead(eng, eng.mtp_weights)
        loop.speculative = SpeculativeDecoder(eng, MtpDraftProvider(head, a.mtp_draft_width), a.mtp_draft_width)
    try:
        svc = GenerationService(loop, tok, eng.cfg.vocab, "cli")
        cfg = GenerationConfig(max_new_tokens=a.max_new_tokens, chain=sampling_from_args(a), seed=a.seed,
                               stop=tuple(a.stop), thinking=a.thinking, separate_reasoning=a.thinking, echo_tokens=True)
        if timeline is not None:
            timeline("PrefillSubmit")
        h = svc.submit(ids, cfg, mm=mm)
        content, reasoning, done, tokens, first = [], [], None, [], True
        for kind, payload in h:
            if kind == "delta":
                if timeline is not None and payload.get("tokens"):
                    if first:
                        timeline("PrefillComplete")
                        timeline("FirstToken")
                        first = False
                    else:
                        timeline("LaterToken")
                tokens += payload.get("tokens", [])
                content.append(payload.get("content", ""))
                reasoning.append(payload.get("reasoning", ""))
                if on_delta:
                    on_delta(payload)
            else:
                done = payload
        if timeline is not None:
            timeline("Stop")
        return "".join(content), "".join(reasoning), done, tokens
    finally:
        loop.shutdown(5.0)
        if timeline is not None:
            timeline("Cleanup")


def _gen_parser(name):
    p = StrictParser(prog=f"sllm {name}")
    add_model_source(p)
    add_generation_args(p)
    return p


def cmd_generate(argv, name="generate"):
    a = _gen_parser(name).parse_args(argv)
    eng, tok, g, lock = open_model(a)
    mm = _multimodal_from_args(eng, tok, a) if a.image else None
    ids = mm.tokens if mm is not None else prompt_ids_from_args(a, tok)
    t0 = time.perf_counter()
    text, reasoning, done, tokens = _generate(eng, tok, ids, a, mm=mm)
    out = {"text": text, "tokens": tokens, "finish_reason": done["finish_reason"], "usage": done["usage"],
           "model": lock["semantic_model_id"], "seconds": round(time.perf_counter() - t0, 4)}
    if reasoning:
        out["reasoning"] = reasoning
    if "error" in done:
        out["error"] = done["error"]
    emit(out)
    return 0 if done["finish_reason"] != "error" else 1


def cmd_completions(argv):
    return cmd_generate(argv, "completions")


def cmd_decode(argv):
    """Greedy continuation of explicit token ids, reported as ids (no tokenizer, no template)."""
    p = StrictParser(prog="sllm decode")
    add_model_source(p)
    p.add_argument("--input-token-ids", required=True)
    p.add_argument("--max-new-tokens", type=int, default=16)
    a = p.parse_args(argv)
    eng, tok, g, lock = open_model(a)
    ids = _parse_ids(a.input_token_ids)
    if not ids or max(ids) >= eng.cfg.vocab:
        raise CliError("token ids must be non-empty and inside the vocabulary")
    out = eng.generate([ids], a.max_new_tokens)[0]
    emit({"input_tokens": ids, "output_tokens": out, "model": lock["semantic_model_id"]})


def cmd_embeddings(argv):
    p = StrictParser(prog="sllm embeddings")
    add_model_source(p)
    p.add_argument("--text", action="append", required=True)
    a = p.parse_args(argv)
    eng, tok, g, lock = open_model(a)
    from ..server.backend import EngineBackend
    b = EngineBackend(eng, tok, aliases=("cli",))
    try:
        vecs = b.embed([tok.encode(t) for t in a.text])
    finally:
        b.shutdown(2.0)
    emit({"embeddings": [[float(x) for x in v] for v in vecs], "dimensions": len(vecs[0])})


def cmd_rerank(argv):
    p = StrictParser(prog="sllm rerank")
    add_model_source(p)
    p.add_argument("--query", required=True)
    p.add_argument("--document", action="append", required=True)
    p.add_argument("--top-n", type=int, default=None)
    a = p.parse_args(argv)
    eng, tok, g, lock = open_model(a)
    from ..server.backend import EngineBackend
    b = EngineBackend(eng, tok, aliases=("cli",))
    try:
        vecs = b.embed([tok.encode(a.query)] + [tok.encode(d) for d in a.document])
    finally:
        b.shutdown(2.0)
    q = vecs[0]
    scored = sorted(((float((q * v).sum()), i) for i, v in enumerate(vecs[1:])), key=lambda t: (-t[0], t[1]))
    if a.top_n:
        scored = scored[:a.top_n]
    emit({"results": [{"index": i, "relevance_score": s} for s, i in scored]})


def cmd_infill(argv):
    p = StrictParser(prog="sllm infill")
    add_model_source(p)
    p.add_argument("--prefix", required=True)
    p.add_argument("--suffix", default="")
    p.add_argument("--max-new-tokens", type=int, default=64)
    p.add_argument("--seed", type=int, default=None)
    a = p.parse_args(argv)
    a.stop, a.thinking, a.prefill_chunk_tokens, a.greedy, a.temperature = [], False, 0, True, None
    eng, tok, g, lock = open_model(a)
    from ..frontend.chat import render_infill
    ids = tok.encode(render_infill(a.prefix, a.suffix))
    text, _, done, tokens = _generate(eng, tok, ids, a)
    emit({"text": text, "finish_reason": done["finish_reason"], "usage": done["usage"]})


def cmd_benchmark(argv):
    p = _gen_parser("benchmark")
    p.add_argument("--lane", choices=("direct", "render"), default="direct")
    p.add_argument("--case-id", default="case")
    p.add_argument("--row-id", default="row")
    p.add_argument("--warmups", type=int, default=1)
    p.add_argument("--measured", type=int, default=3)
    p.add_argument("--model-size", default="")
    a = p.parse_args(argv)
    eng, tok, g, lock = open_model(a)
    ids = prompt_ids_from_args(a, tok)
    schema = BENCH_SCHEMA_DIRECT if a.lane == "direct" else BENCH_SCHEMA_RENDER
    for it in range(a.warmups + a.measured):
        measured = it >= a.warmups
        t0 = time.perf_counter()
        events = []
        tl = lambda name: events.append({"event": name, "t_ms": round((time.perf_counter() - t0) * 1e3, 3)})
        text, _, done, tokens = _generate(eng, tok, ids, a, timeline=tl)
        by = {}
        for e in events:
            by.setdefault(e["event"], e["t_ms"])
        later = [e["t_ms"] for e in events if e["event"] == "LaterToken"]
        n = done["usage"]["completion_tokens"]
        first = by.get("FirstToken", 0.0)
        last = later[-1] if later else first
        emit({"schema": schema, "case_id": a.case_id, "row_id": a.row_id, "model_size": a.model_size, "lane": a.lane,
              "iteration": it, "measured": measured, "prompt_tokens": len(ids), "completion_tokens": n,
              "ttft_ms": first, "decode_tok_s": round((n - 1) / ((last - first) / 1e3), 3) if n > 1 and last > first else None,
              "total_ms": by.get("Stop"), "finish_reason": done["finish_reason"], "timeline": events})


def cmd_chat(argv):
    from .chat import run_chat
    return run_chat(argv)


def cmd_models(argv):
    from .model_admin import run_models
    return run_models(argv)


DISPATCH = {"version": cmd_version, "doctor": cmd_doctor, "chat": cmd_chat, "models": cmd_models,
            "verify-model": cmd_verify_model, "tokenize": cmd_tokenize, "detokenize": cmd_detokenize,
            "render": cmd_render, "apply-template": cmd_apply_template, "input-tokens": cmd_input_tokens,
            "completions": cmd_completions, "embeddings": cmd_embeddings, "rerank": cmd_rerank, "infill": cmd_infill,
            "decode": cmd_decode, "generate": cmd_generate, "benchmark": cmd_benchmark}


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)

    def go():
        if not argv or argv[0] in ("-h", "--help", "help"):
            emit({"usage": "sllm <command> [flags]", "commands": list(COMMANDS)})
            return 0 if argv else 2
        cmd = DISPATCH.get(argv[0])
        if cmd is None:
            raise CliError(f"unknown command {argv[0]!r}; commands: {', '.join(COMMANDS)}")
        return cmd(argv[1:])

    return run_main(go)


if __name__ == "__main__":
    sys.exit(main())

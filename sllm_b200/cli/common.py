"""Shared pieces of the command-line tools: the model source, strict argument parsing, JSON output.

Every command that runs a model takes `--gguf PATH --derived-lock PATH --device-index N --target sm_100a`
(reference: crates/sllm-cli/src/main.rs:70-73; the AMD target name becomes the one CUDA target).  The file is
verified against its derived lock before any tensor is read, and the same descriptor serves the upload.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Optional

TARGET = "sm_100a"
KV_ENCODINGS = ("fp16", "bf16", "fp8", "fp8-static", "nvfp4")


class CliError(Exception):
    def __init__(self, message: str, code: int = 2):
        super().__init__(message)
        self.code = code


class StrictParser(argparse.ArgumentParser):
    """No abbreviations, errors as exceptions (the commands print one JSON error line and exit 2)."""

    def __init__(self, *a, **kw):
        kw.setdefault("allow_abbrev", False)
        kw.setdefault("add_help", True)
        super().__init__(*a, **kw)

    def error(self, message):
        raise CliError(message, 2)


def add_model_source(p: argparse.ArgumentParser, required: bool = True) -> None:
    p.add_argument("--gguf", required=required)
    p.add_argument("--derived-lock", required=required)
    p.add_argument("--device-index", type=int, default=0)
    p.add_argument("--target", default=TARGET)
    p.add_argument("--kv-cache-encoding", choices=KV_ENCODINGS, default=None)
    p.add_argument("--context-length", type=int, default=None)
    p.add_argument("--activation-encoding", choices=ACT_ENCODINGS, default=None,
                   help="4-bit-weight models: bf16 (W4A16, default) or fp4 (activations quantised to the weights' 4-bit "
                        "format, GEMMs on the block-scaled tensor-core kernel)")
    p.add_argument("--cpu", action="store_true", help="run the CPU oracle path (small models only)")


def emit(obj) -> None:
    sys.stdout.write(json.dumps(obj, ensure_ascii=False, separators=(",", ":")) + "\n")
    sys.stdout.flush()


ACT_ENCODINGS = ("bf16", "fp4")


def apply_activation_encoding(args) -> None:
    enc = getattr(args, "activation_encoding", None)
    if enc is not None:
        from ..ops import w4
        w4.set_w4a4(enc == "fp4")


_KV_MAP = {"fp16": "bf16", "bf16": "bf16", "fp8": "fp8", "fp8-static": "fp8-static", "nvfp4": "nvfp4"}


def open_model(args, max_batch: int = 8, tp=None):
    """Returns (engine, tokenizer, gguf_file, lock).  Raises CliError with a user-facing message."""
    import torch
    from ..cache.paged import PagedKVCache
    from ..engine.engine import Engine
    from ..formats import gguf as G
    from ..models import loader
    from ..models.llama import LlamaModel
    if args.target != TARGET:
        raise CliError(f"unsupported target {args.target!r}: this build runs on {TARGET} only")
    try:
        lock = G.read_derived_lock(args.derived_lock)
        g = G.verify_gguf(args.gguf, lock)
    except (OSError, G.GgufError) as exc:
        raise CliError(f"model verification failed: {exc}", 3) from None
    apply_activation_encoding(args)
    use_cpu = getattr(args, "cpu", False)
    if not use_cpu and not torch.cuda.is_available():
        raise CliError("no CUDA device is available (pass --cpu for the CPU oracle path)", 4)
    device = torch.device("cpu") if use_cpu else torch.device("cuda", args.device_index)
    kvf = None
    if args.kv_cache_encoding:
        kvf = _KV_MAP[args.kv_cache_encoding]
    tp_size, tp_rank = (tp.size, tp.rank) if tp is not None else (1, 0)
    ep = getattr(args, "_ep", None)           # expert-parallel context of a mixture-of-experts run (same ranks as tp)
    ep_size, ep_rank = (ep.size, ep.rank) if ep is not None else (1, 0)
    try:
        cfg, weights, family = loader.load_model_gguf(g, device, tp_size, tp_rank, ep_size, ep_rank, kv_format=kvf)
    except G.GgufError as exc:
        raise CliError(f"model load failed: {exc}", 3) from None
    if use_cpu and cfg.kv_format not in ("fp32", "bf16", "nvfp4"):
        cfg.kv_format = "fp32"
    if args.context_length:
        if args.context_length > cfg.max_context:
            emit({"event": "warning", "code": "context_length_exceeds_recommended",
                  "requested": args.context_length, "recommended": cfg.max_context})
        cfg.max_context = args.context_length
    blocks = (cfg.max_context + cfg.page_size - 1) // cfg.page_size
    if family == "moe":
        from ..models.moe import MoeModel
        model = MoeModel(cfg, weights, tp, ep)
        cache = PagedKVCache(cfg, max_batch * blocks + 8, device, kv_heads=model.local_kv_heads)
    elif family == "qwen35":
        from ..cache.hybrid import HybridCache
        from ..models.qwen35 import Qwen35Model
        model = Qwen35Model(cfg, weights, tp, ep)
        cache = HybridCache(cfg, max_batch * blocks + 8, device, max_seqs=2 * max_batch + 2, kv_heads=model.local_kv_heads,
                            tp_size=tp_size)
    else:
        model = LlamaModel(cfg, weights, tp)
        cache = PagedKVCache(cfg, max_batch * blocks + 8, device, kv_heads=model.local_kv_heads)
    eng = Engine(cfg, model, cache, device, max_batch=max_batch, use_cuda_graphs=not use_cpu, tp=tp)
    dense_family = family not in ("moe", "qwen35")
    eng.mtp_weights = loader.load_mtp_gguf(g, cfg, device) if tp_size == 1 and dense_family else None
    vis = loader.load_vision_gguf(g, cfg, device) if dense_family else None
    if vis is not None:
        from ..models.vision_tower import VisionTower
        eng.vision = VisionTower(*vis)
    tok = loader.tokenizer_from_gguf(g)
    return eng, tok, g, lock


def sampling_from_args(args):
    from ..engine import sampling as S
    greedy = getattr(args, "greedy", False) or getattr(args, "temperature", None) in (None, 0.0)
    params = S.SamplingParams(temperature=0.0 if greedy else args.temperature, top_p=getattr(args, "top_p", 1.0) or 1.0,
                              presence_penalty=getattr(args, "presence_penalty", 0.0) or 0.0,
                              frequency_penalty=getattr(args, "frequency_penalty", 0.0) or 0.0)
    return S.SamplerChainConfig(params=params)


def add_generation_args(p: argparse.ArgumentParser) -> None:
    p.add_argument("--prompt")
    p.add_argument("--message", action="append", default=[], metavar="ROLE:CONTENT")
    p.add_argument("--input-token-ids")
    p.add_argument("--max-new-tokens", type=int, default=128)
    p.add_argument("--greedy", action="store_true")
    p.add_argument("--temperature", type=float, default=None)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--presence-penalty", type=float, default=0.0)
    p.add_argument("--frequency-penalty", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=None)
    p.add_argument("--stop", action="append", default=[])
    p.add_argument("--image", action="append", default=[])
    p.add_argument("--thinking", action="store_true")
    p.add_argument("--prefill-chunk-tokens", type=int, default=0)
    p.add_argument("--mtp-draft-width", type=int, default=0)
    p.add_argument("--no-generation-prompt", action="store_true")


def prompt_ids_from_args(args, tok, as_text: bool = False):
    """Token ids of the request (or, with as_text, its rendered text; --image inputs put one vision marker each in
    front of the first user message)."""
    from ..frontend.chat import ChatMessage, render_chatml
    given = [x for x in (args.prompt, args.message or None, args.input_token_ids) if x]
    if len(given) != 1:
        raise CliError("give exactly one of --prompt, --message or --input-token-ids")
    if len(args.stop) > 4:
        raise CliError("at most 4 --stop strings")
    if len(args.image) > 2:
        raise CliError("at most 2 --image inputs")
    if not 0 <= args.mtp_draft_width <= 8:
        raise CliError("--mtp-draft-width must be in 0..8")
    if args.input_token_ids:
        try:
            ids = [int(x) for x in args.input_token_ids.replace(",", " ").split()]
        except ValueError:
            raise CliError("--input-token-ids must be integers") from None
        if not ids or any(i < 0 for i in ids):
            raise CliError("--input-token-ids must be non-negative and non-empty")
        if as_text:
            raise CliError("--image needs --prompt or --message")
        return ids
    if args.prompt is not None:
        msgs = [ChatMessage("user", args.prompt)]
    else:
        msgs = []
        for m in args.message:
            role, sep, content = m.partition(":")
            if not sep or role not in ("system", "user", "assistant", "tool"):
                raise CliError("--message must look like ROLE:CONTENT with role system|user|assistant|tool")
            msgs.append(ChatMessage(role, content))
    if args.image:
        marks = "<|vision_start|><|image_pad|><|vision_end|>" * len(args.image)
        for i, m in enumerate(msgs):
            if m.role == "user":
                msgs[i] = ChatMessage("user", marks + m.content)
                break
        else:
            raise CliError("--image needs a user message")
    text = render_chatml(msgs, thinking="enabled" if args.thinking else "disabled",
                         add_generation_prompt=not args.no_generation_prompt)
    return text if as_text else tok.encode(text)


def run_main(fn) -> int:
    try:
        return fn() or 0
    except CliError as exc:
        emit({"event": "error", "message": str(exc)})
        return exc.code
    except KeyboardInterrupt:
        emit({"event": "error", "message": "interrupted"})
        return 130

"""Strict request parsers for every wire profile: unknown field -> 400, no silent coercion, explicit
ranges and limits.

Profiles (reference: docs/api/openai-compatibility.md, docs/api/anthropic-compatibility.md,
crates/sllm-server/src/api.rs:771-786, phase42_api.rs, phase43_api.rs):
  * Chat Completions profile v1 (+ `sllm` extension object, + openwebui compatibility profile)
  * Completions, Embeddings, Rerank, Tokenize / Detokenize / Apply-template / Input-tokens, Infill
  * Responses, Anthropic Messages (text + client-side function tools)
"""
from __future__ import annotations

import base64
import math
from dataclasses import dataclass, field
from typing import Optional

from ..engine import sampling as S
from ..frontend.chat import ChatMessage
from . import errors as E

MAX_BODY_BYTES = 96 * 1024 * 1024
MAX_ALIAS_BYTES = 256
MAX_MESSAGES = 1024
MAX_COMPLETION_TOKENS = 4096
MAX_N = 8
MAX_STOP = 4
MAX_IMAGES = 2
MAX_RERANK_DOCS = 256
MAX_INPUTS = 2048

_CHAT_FIELDS = {"model", "messages", "temperature", "top_p", "max_completion_tokens", "stop", "presence_penalty",
                "frequency_penalty", "seed", "stream", "n", "logit_bias", "logprobs", "top_logprobs",
                "response_format", "sllm", "tools", "tool_choice"}
_KNOWN_UNSUPPORTED_CHAT = {"functions", "function_call", "audio", "modalities", "prediction", "store", "metadata",
                           "service_tier", "parallel_tool_calls", "stream_options", "user", "reasoning_effort",
                           "web_search_options", "max_tokens"}
_SLLM_FIELDS = {"sampling", "thinking", "separate_reasoning", "resumable", "adapters", "control_vectors",
                "reasoning_budget"}
_SAMPLING_FIELDS = {"chain_version", "top_k", "min_p", "typical_p", "repeat_penalty", "repeat_last_n", "ignore_eos",
                    "dry", "xtc", "mirostat", "dynamic_temperature"}


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool) and math.isfinite(v)


def _require_obj(v, param):
    if not isinstance(v, dict):
        raise E.invalid_value(f"{param} must be an object", param)
    return v


def _check_fields(obj: dict, allowed: set, known_unsupported: set = frozenset(), prefix: str = ""):
    for k in obj:
        if k in allowed:
            continue
        if k in known_unsupported:
            raise E.unsupported(f"{prefix}{k} is not supported by this profile", prefix + k)
        raise E.unsupported(f"unknown field {prefix}{k}", prefix + k)


def _model(obj) -> str:
    m = obj.get("model")
    if not isinstance(m, str) or not m:
        raise E.invalid_value("model must be a non-empty string", "model")
    if len(m.encode("utf-8")) > MAX_ALIAS_BYTES:
        raise E.invalid_value("model alias longer than 256 bytes", "model")
    return m


def _num_in(obj, key, lo, hi, default):
    if key not in obj or obj[key] is None:
        return default
    v = obj[key]
    if not _is_num(v) or not lo <= v <= hi:
        raise E.invalid_value(f"{key} must be a finite number in [{lo}, {hi}]", key)
    return float(v)


def _int_in(obj, key, lo, hi, default, param=None):
    if key not in obj or obj[key] is None:
        return default
    v = obj[key]
    if not _is_int(v) or not lo <= v <= hi:
        raise E.invalid_value(f"{param or key} must be an integer in {lo}..{hi}", param or key)
    return v


def _bool(obj, key, default=False):
    if key not in obj or obj[key] is None:
        return default
    if not isinstance(obj[key], bool):
        raise E.invalid_value(f"{key} must be a boolean", key)
    return obj[key]


def _stop(obj, key="stop") -> tuple:
    if key not in obj or obj[key] is None:
        return ()
    v = obj[key]
    if isinstance(v, str):
        v = [v]
    if not isinstance(v, list) or not 1 <= len(v) <= MAX_STOP or any(not isinstance(s, str) or not s for s in v) \
            or len(set(v)) != len(v):
        raise E.invalid_value("stop must be a string or an array of 1-4 unique non-empty strings", key)
    return tuple(v)


def _seed(obj):
    if "seed" not in obj or obj["seed"] is None:
        return None
    v = obj["seed"]
    if not _is_int(v) or not -(1 << 63) <= v < (1 << 63):
        raise E.invalid_value("seed must be a signed 64-bit integer", "seed")
    return v & ((1 << 64) - 1)


def _logit_bias(obj) -> list:
    lb = obj.get("logit_bias")
    if lb is None:
        return []
    _require_obj(lb, "logit_bias")
    if len(lb) > S.MAX_LOGIT_BIAS:
        raise E.invalid_value("logit_bias holds more than 4096 entries", "logit_bias")
    out = []
    for k, v in lb.items():
        if not (isinstance(k, str) and k.isdigit() and (k == "0" or not k.startswith("0"))):
            raise E.invalid_value("logit_bias keys must be decimal token ids", "logit_bias")
        if not _is_num(v) or not -100 <= v <= 100:
            raise E.invalid_value("logit_bias values must be finite numbers in [-100, 100]", "logit_bias")
        out.append((int(k), float(v)))
    return out


@dataclass
class ImagePart:
    mime: str
    data: bytes


@dataclass
class ParsedSampling:
    chain: S.SamplerChainConfig
    seed: Optional[int]


def _sampling_extension(ext: Optional[dict], chain: S.SamplerChainConfig) -> None:
    if ext is None:
        return
    _require_obj(ext, "sllm.sampling")
    _check_fields(ext, _SAMPLING_FIELDS, prefix="sllm.sampling.")
    if ext.get("chain_version", 1) != 1:
        raise E.invalid_value("sllm.sampling.chain_version must be 1", "sllm.sampling.chain_version")
    tk = _int_in(ext, "top_k", 0, 1_000_000, 0, "sllm.sampling.top_k")
    chain.top_k = tk or None
    chain.min_p = _num_in(ext, "min_p", 0.0, 1.0, 0.0)
    tp = _num_in(ext, "typical_p", 0.0, 1.0, 1.0)
    if tp <= 0:
        raise E.invalid_value("sllm.sampling.typical_p must be in (0, 1]", "sllm.sampling.typical_p")
    chain.typical_p = tp
    rp = _num_in(ext, "repeat_penalty", 0.0, 100.0, 1.0)
    if rp <= 0 or rp > 10:
        raise E.invalid_value("sllm.sampling.repeat_penalty must be in (0, 10]", "sllm.sampling.repeat_penalty")
    chain.repeat_penalty = rp
    chain.repeat_last_n = _int_in(ext, "repeat_last_n", 0, 4096, 64, "sllm.sampling.repeat_last_n")
    chain._ignore_eos = _bool(ext, "ignore_eos")
    try:
        if ext.get("dry") is not None:
            d = _require_obj(ext["dry"], "sllm.sampling.dry")
            _check_fields(d, {"multiplier", "base", "allowed_length", "penalty_last_n", "sequence_breakers"},
                          prefix="sllm.sampling.dry.")
            br = d.get("sequence_breakers", [])
            if not isinstance(br, list) or len(br) > 16 or any(not isinstance(b, str) or not b for b in br) \
                    or len(set(br)) != len(br) or sum(len(b.encode()) for b in br) > 1024:
                raise E.invalid_value("dry.sequence_breakers: at most 16 unique strings, 1024 bytes in total",
                                      "sllm.sampling.dry.sequence_breakers")
            chain._dry_raw = (float(d.get("multiplier", 0.0)), float(d.get("base", 1.75)),
                              int(d.get("allowed_length", 2)), int(d.get("penalty_last_n", S.MAX_SAMPLING_HISTORY)), br)
            S.DryConfig(chain._dry_raw[0], chain._dry_raw[1], chain._dry_raw[2], [], chain._dry_raw[3])
        if ext.get("xtc") is not None:
            x = _require_obj(ext["xtc"], "sllm.sampling.xtc")
            _check_fields(x, {"probability", "threshold", "min_keep"}, prefix="sllm.sampling.xtc.")
            chain.xtc = S.XtcConfig(float(x.get("probability", 0.0)), float(x.get("threshold", 0.1)),
                                    int(x.get("min_keep", 1)))
        if ext.get("mirostat") is not None:
            m = _require_obj(ext["mirostat"], "sllm.sampling.mirostat")
            _check_fields(m, {"version", "tau", "eta"}, prefix="sllm.sampling.mirostat.")
            tau, eta = float(m.get("tau", 5.0)), float(m.get("eta", 0.1))
            if not 0 < tau <= 100 or not 0 < eta <= 1:
                raise E.invalid_value("mirostat tau must be in (0,100] and eta in (0,1]", "sllm.sampling.mirostat")
            if chain.top_k or chain.min_p or chain.typical_p < 1 or chain.xtc or ext.get("dynamic_temperature"):
                raise E.invalid_value("mirostat cannot be combined with top_k, min_p, typical_p, xtc or dynamic "
                                      "temperature", "sllm")
            chain.mirostat = S.MirostatConfig(int(m.get("version", 2)), tau, eta, 2 * tau)
        if ext.get("dynamic_temperature") is not None:
            dt = _require_obj(ext["dynamic_temperature"], "sllm.sampling.dynamic_temperature")
            _check_fields(dt, {"range", "exponent"}, prefix="sllm.sampling.dynamic_temperature.")
            chain.dynamic_temperature = (float(dt.get("range", 0.0)), float(dt.get("exponent", 1.0)))
        chain.validate()
    except S.SamplingError as exc:
        raise E.invalid_value(str(exc), "sllm.sampling") from None
    except (TypeError, ValueError) as exc:
        if isinstance(exc, E.ApiError):
            raise
        raise E.invalid_value("invalid sllm.sampling member", "sllm.sampling") from None


def _common_sampling(obj, max_tokens_key: str, compat_openwebui: bool = False):
    try:
        params = S.SamplingParams(_num_in(obj, "temperature", 0.0, 2.0, 1.0), _num_in(obj, "top_p", 0.0, 1.0, 1.0),
                                  _num_in(obj, "presence_penalty", -2.0, 2.0, 0.0),
                                  _num_in(obj, "frequency_penalty", -2.0, 2.0, 0.0))
    except S.SamplingError as exc:
        raise E.invalid_value(str(exc)) from None
    chain = S.SamplerChainConfig(params=params, logit_bias=_logit_bias(obj))
    return chain


@dataclass
class ChatRequest:
    model: str
    messages: list
    images: list
    chain: S.SamplerChainConfig
    seed: Optional[int]
    max_tokens: int
    stop: tuple
    stream: bool
    n: int
    logprobs: bool
    response_format: dict
    thinking: bool
    separate_reasoning: bool
    reasoning_budget: Optional[int]
    resumable: bool
    ignore_eos: bool
    adapters: list
    control_vectors: list
    tools: list
    tool_choice: object
    dry_breakers: list = field(default_factory=list)


def _parse_content(role: str, content, images: list, idx: int, multimodal: bool = True) -> str:
    if isinstance(content, str):
        return content
    if not multimodal:
        raise E.unsupported("multipart content is outside this profile", f"messages[{idx}].content")
    if role != "user" or not isinstance(content, list) or not content:
        raise E.invalid_value("content must be a string (multipart content is limited to user messages)",
                              f"messages[{idx}].content")
    texts = []
    for part in content:
        if not isinstance(part, dict):
            raise E.invalid_value("content parts must be objects", f"messages[{idx}].content")
        t = part.get("type")
        if t == "text":
            _check_fields(part, {"type", "text"}, prefix=f"messages[{idx}].content.")
            if not isinstance(part.get("text"), str) or not part["text"]:
                raise E.invalid_value("text parts must be non-empty strings", f"messages[{idx}].content")
            texts.append(part["text"])
        elif t == "image_url":
            _check_fields(part, {"type", "image_url"}, prefix=f"messages[{idx}].content.")
            iu = _require_obj(part.get("image_url"), f"messages[{idx}].content.image_url")
            _check_fields(iu, {"url", "detail"}, prefix=f"messages[{idx}].content.image_url.")
            if iu.get("detail", "auto") != "auto":
                raise E.unsupported("image detail must be omitted or auto", f"messages[{idx}].content.image_url.detail")
            url = iu.get("url")
            if not isinstance(url, str) or not url.startswith("data:image/") or ";base64," not in url:
                raise E.unsupported("only base64 data URLs are accepted for images",
                                    f"messages[{idx}].content.image_url.url")
            mime, b64 = url[5:].split(";base64,", 1)
            if mime not in ("image/png", "image/jpeg", "image/webp", "image/gif"):
                raise E.unsupported("unsupported image type", f"messages[{idx}].content.image_url.url")
            try:
                data = base64.b64decode(b64, validate=True)
            except Exception:
                raise E.invalid_value("image data is not valid base64", f"messages[{idx}].content.image_url.url") from None
            if any(i.data == data for i in images):
                raise E.invalid_value("duplicate image", f"messages[{idx}].content")
            images.append(ImagePart(mime, data))
            if len(images) > MAX_IMAGES:
                raise E.invalid_value("at most two images per request", f"messages[{idx}].content")
            texts.append("<|vision_start|><|image_pad|><|vision_end|>")
        else:
            raise E.unsupported("unsupported content part type", f"messages[{idx}].content")
    return "".join(texts)


def parse_chat_request(obj, compat_openwebui: bool = False, multimodal: bool = False) -> ChatRequest:
    _require_obj(obj, "body")
    allowed = set(_CHAT_FIELDS) | ({"max_tokens"} if compat_openwebui else set())
    _check_fields(obj, allowed, _KNOWN_UNSUPPORTED_CHAT)
    model = _model(obj)
    msgs_raw = obj.get("messages")
    if not isinstance(msgs_raw, list) or not msgs_raw:
        raise E.invalid_value("messages must be a non-empty array", "messages")
    if len(msgs_raw) > MAX_MESSAGES:
        raise E.invalid_value("too many messages", "messages")
    messages, images = [], []
    for i, m in enumerate(msgs_raw):
        _require_obj(m, f"messages[{i}]")
        role = m.get("role")
        if role in ("developer", "tool", "function"):
            raise E.unsupported(f"role {role} is outside this profile", f"messages[{i}].role")
        if role not in ("system", "user", "assistant"):
            raise E.invalid_value("role must be system, user or assistant", f"messages[{i}].role")
        _check_fields(m, {"role", "content"} | ({"reasoning_content"} if role == "assistant" else set()),
                      {"name", "tool_calls", "tool_call_id", "function_call", "audio", "refusal"},
                      prefix=f"messages[{i}].")
        content = _parse_content(role, m.get("content"), images, i, multimodal)
        rc = m.get("reasoning_content")
        if rc is not None and not isinstance(rc, str):
            raise E.invalid_value("reasoning_content must be a string", f"messages[{i}].reasoning_content")
        messages.append(ChatMessage(role, content, rc))
    if sum(1 for m in messages if m.role == "system") > 1 or any(m.role == "system" and i for i, m in enumerate(messages)):
        raise E.invalid_value("at most one system message, and it must be first", "messages")
    if not any(m.role == "user" for m in messages):
        raise E.invalid_value("at least one user message is required", "messages")

    chain = _common_sampling(obj, "max_completion_tokens")
    if compat_openwebui and "max_tokens" in obj:
        if "max_completion_tokens" in obj:
            raise E.invalid_value("send only one of max_tokens and max_completion_tokens", "max_tokens")
        max_tokens = _int_in(obj, "max_tokens", 1, MAX_COMPLETION_TOKENS, 256)
    else:
        max_tokens = _int_in(obj, "max_completion_tokens", 1, MAX_COMPLETION_TOKENS, 256)
    logprobs = _bool(obj, "logprobs")
    top_lp = _int_in(obj, "top_logprobs", 0, 20, 0)
    if top_lp and not logprobs:
        raise E.invalid_value("top_logprobs requires logprobs: true", "top_logprobs")
    chain.return_logprobs, chain.top_logprobs = logprobs, top_lp
    stream = _bool(obj, "stream")
    n = _int_in(obj, "n", 1, MAX_N, 1)

    rf = obj.get("response_format") or {"type": "text"}
    _require_obj(rf, "response_format")
    if rf.get("type") not in ("text", "json_object", "json_schema"):
        raise E.invalid_value("response_format.type must be text, json_object or json_schema", "response_format.type")
    if rf["type"] == "json_object":
        _check_fields(rf, {"type"}, prefix="response_format.")
        if not any("json" in m.content.lower() for m in messages):
            raise E.invalid_value("json_object requires a message that mentions JSON", "response_format")
    elif rf["type"] == "json_schema":
        _check_fields(rf, {"type", "json_schema"}, prefix="response_format.")
        js = _require_obj(rf.get("json_schema"), "response_format.json_schema")
        _check_fields(js, {"name", "description", "strict", "schema"}, prefix="response_format.json_schema.")
        if not isinstance(js.get("name"), str) or not 0 < len(js["name"].encode()) <= 256:
            raise E.invalid_value("json_schema.name must be 1-256 bytes", "response_format.json_schema.name")
        if js.get("description") is not None and (not isinstance(js["description"], str) or len(js["description"].encode()) > 4096):
            raise E.invalid_value("json_schema.description too long", "response_format.json_schema.description")
        if js.get("strict") is not None and not isinstance(js["strict"], bool):
            raise E.invalid_value("json_schema.strict must be a boolean", "response_format.json_schema.strict")
        _require_obj(js.get("schema"), "response_format.json_schema.schema")
    else:
        _check_fields(rf, {"type"}, prefix="response_format.")

    ext = obj.get("sllm")
    thinking = separate = resumable = ignore_eos = False
    budget = None
    adapters, cvs, dry_breakers = [], [], []
    if ext is not None:
        _require_obj(ext, "sllm")
        _check_fields(ext, _SLLM_FIELDS, prefix="sllm.")
        _sampling_extension(ext.get("sampling"), chain)
        ignore_eos = getattr(chain, "_ignore_eos", False)
        if hasattr(chain, "_dry_raw"):
            dry_breakers = chain._dry_raw[4]
        th = ext.get("thinking", "disabled")
        if th not in ("enabled", "disabled", "template-default"):
            raise E.invalid_value("sllm.thinking must be enabled, disabled or template-default", "sllm.thinking")
        thinking = th == "enabled"
        separate = _bool(ext, "separate_reasoning")
        if separate and not thinking:
            raise E.invalid_value("separate_reasoning requires thinking: enabled", "sllm.separate_reasoning")
        budget = _int_in(ext, "reasoning_budget", 1, 4096, None, "sllm.reasoning_budget")
        if budget is not None and not thinking:
            raise E.invalid_value("reasoning_budget requires thinking: enabled", "sllm.reasoning_budget")
        resumable = _bool(ext, "resumable")
        if resumable and not stream:
            raise E.invalid_value("sllm.resumable requires stream: true", "sllm.resumable")
        adapters = _artifact_selection(ext.get("adapters"), "sllm.adapters")
        cvs = _artifact_selection(ext.get("control_vectors"), "sllm.control_vectors")
        if {a for a, _ in adapters} & {c for c, _ in cvs}:
            raise E.invalid_value("an artifact name may appear in only one list", "sllm")
    tools, tool_choice = [], None
    if "tools" in obj or "tool_choice" in obj:
        raise E.unsupported("tools are outside Chat Completions profile v1; use /v1/responses or /v1/messages", "tools")
    try:
        chain.validate()
    except S.SamplingError as exc:
        raise E.invalid_value(str(exc)) from None
    return ChatRequest(model, messages, images, chain, _seed(obj), max_tokens, _stop(obj), stream, n, logprobs, rf,
                       thinking, separate, budget, resumable, ignore_eos, adapters, cvs, tools, tool_choice, dry_breakers)


def _artifact_selection(raw, param) -> list:
    if raw is None:
        return []
    if not isinstance(raw, list) or len(raw) > 4:
        raise E.invalid_value(f"{param} must be an array of at most four entries", param)
    out = []
    for e in raw:
        if isinstance(e, str):
            name, scale = e, 1.0
        elif isinstance(e, dict):
            _check_fields(e, {"name", "scale"}, prefix=param + ".")
            name, scale = e.get("name"), e.get("scale", 1.0)
        else:
            raise E.invalid_value(f"{param} entries must be names or objects", param)
        if not isinstance(name, str) or not name or not _is_num(scale) or not -16 <= scale <= 16:
            raise E.invalid_value(f"{param}: name required, scale in [-16, 16]", param)
        out.append((name, float(scale)))
    names = [n for n, _ in out]
    if len(set(names)) != len(names) or names != sorted(names):
        raise E.invalid_value(f"{param} must be unique and in canonical (sorted) order", param)
    return out


# ------------------------------------------------------------------------------------------------ completions
@dataclass
class CompletionRequest:
    model: str
    prompts: list          # list of str or list[int]
    chain: S.SamplerChainConfig
    seed: Optional[int]
    max_tokens: int
    stop: tuple
    stream: bool
    n: int
    echo: bool
    logprobs: int


def _prompt_shapes(v, param) -> list:
    if isinstance(v, str):
        return [v]
    if isinstance(v, list) and v:
        if all(isinstance(x, str) for x in v):
            return list(v)
        if all(_is_int(x) and x >= 0 for x in v):
            return [list(v)]
        if all(isinstance(x, list) and x and all(_is_int(t) and t >= 0 for t in x) for x in v):
            return [list(x) for x in v]
    raise E.invalid_value(f"{param} must be a string, string array, token array or array of token arrays", param)


def parse_completion_request(obj) -> CompletionRequest:
    _require_obj(obj, "body")
    _check_fields(obj, {"model", "prompt", "max_tokens", "temperature", "top_p", "n", "stream", "stop", "seed",
                        "presence_penalty", "frequency_penalty", "logit_bias", "logprobs", "echo"},
                  {"best_of", "suffix", "user", "stream_options"})
    prompts = _prompt_shapes(obj.get("prompt"), "prompt")
    if len(prompts) > MAX_INPUTS:
        raise E.invalid_value("too many prompts", "prompt")
    chain = _common_sampling(obj, "max_tokens")
    lp = _int_in(obj, "logprobs", 0, 5, None)
    if lp is not None:
        chain.return_logprobs, chain.top_logprobs = True, lp
    return CompletionRequest(_model(obj), prompts, chain, _seed(obj), _int_in(obj, "max_tokens", 1, MAX_COMPLETION_TOKENS, 16),
                             _stop(obj), _bool(obj, "stream"), _int_in(obj, "n", 1, MAX_N, 1), _bool(obj, "echo"), lp or 0)


@dataclass
class EmbeddingRequest:
    model: str
    inputs: list
    encoding_format: str
    dimensions: Optional[int]


def parse_embedding_request(obj) -> EmbeddingRequest:
    _require_obj(obj, "body")
    _check_fields(obj, {"model", "input", "encoding_format", "dimensions"}, {"user"})
    inputs = _prompt_shapes(obj.get("input"), "input")
    if len(inputs) > MAX_INPUTS or any((isinstance(x, str) and not x) for x in inputs):
        raise E.invalid_value("input must hold 1-2048 non-empty items", "input")
    fmt = obj.get("encoding_format", "float")
    if fmt not in ("float", "base64"):
        raise E.invalid_value("encoding_format must be float or base64", "encoding_format")
    if obj.get("dimensions") is not None:
        raise E.unsupported("dimensions is fixed by the model", "dimensions")
    return EmbeddingRequest(_model(obj), inputs, fmt, None)


@dataclass
class RerankRequest:
    model: str
    query: str
    documents: list
    top_n: int
    return_documents: bool


def parse_rerank_request(obj) -> RerankRequest:
    _require_obj(obj, "body")
    _check_fields(obj, {"model", "query", "documents", "top_n", "return_documents"})
    q, docs = obj.get("query"), obj.get("documents")
    if not isinstance(q, str) or not q:
        raise E.invalid_value("query must be a non-empty string", "query")
    if not isinstance(docs, list) or not 1 <= len(docs) <= MAX_RERANK_DOCS or any(not isinstance(d, str) or not d for d in docs):
        raise E.invalid_value("documents must hold 1-256 non-empty strings", "documents")
    return RerankRequest(_model(obj), q, docs, _int_in(obj, "top_n", 1, len(docs), len(docs)), _bool(obj, "return_documents"))


def parse_tokenize_request(obj):
    _require_obj(obj, "body")
    _check_fields(obj, {"model", "content", "add_special", "with_pieces"})
    if not isinstance(obj.get("content"), str):
        raise E.invalid_value("content must be a string", "content")
    return _model(obj), obj["content"], _bool(obj, "add_special", True), _bool(obj, "with_pieces")


def parse_detokenize_request(obj):
    _require_obj(obj, "body")
    _check_fields(obj, {"model", "tokens", "skip_special_tokens"})
    t = obj.get("tokens")
    if not isinstance(t, list) or any(not _is_int(x) or x < 0 for x in t) or len(t) > 1_048_576:
        raise E.invalid_value("tokens must be an array of non-negative integers", "tokens")
    return _model(obj), t, _bool(obj, "skip_special_tokens")


def _simple_messages(raw, param="messages") -> list:
    if not isinstance(raw, list) or not raw or len(raw) > MAX_MESSAGES:
        raise E.invalid_value("messages must be a non-empty array", param)
    out = []
    for i, m in enumerate(raw):
        _require_obj(m, f"{param}[{i}]")
        _check_fields(m, {"role", "content", "reasoning_content"}, prefix=f"{param}[{i}].")
        if m.get("role") not in ("system", "user", "assistant") or not isinstance(m.get("content"), str):
            raise E.invalid_value("messages need a role (system, user, assistant) and string content", f"{param}[{i}]")
        out.append(ChatMessage(m["role"], m["content"], m.get("reasoning_content")))
    return out


def parse_apply_template_request(obj):
    _require_obj(obj, "body")
    _check_fields(obj, {"model", "messages", "add_generation_prompt", "thinking"})
    th = obj.get("thinking", "disabled")
    if th not in ("enabled", "disabled", "template-default"):
        raise E.invalid_value("thinking must be enabled, disabled or template-default", "thinking")
    return _model(obj), _simple_messages(obj.get("messages")), _bool(obj, "add_generation_prompt", True), th


def parse_infill_request(obj):
    _require_obj(obj, "body")
    _check_fields(obj, {"model", "input_prefix", "input_suffix", "max_tokens", "temperature", "top_p", "seed", "stop",
                        "stream", "presence_penalty", "frequency_penalty", "logit_bias"})
    p, s = obj.get("input_prefix"), obj.get("input_suffix")
    if not isinstance(p, str) or not isinstance(s, str):
        raise E.invalid_value("input_prefix and input_suffix must be strings", "input_prefix")
    return (_model(obj), p, s, _common_sampling(obj, "max_tokens"), _seed(obj),
            _int_in(obj, "max_tokens", 1, MAX_COMPLETION_TOKENS, 64), _stop(obj), _bool(obj, "stream"))


# ------------------------------------------------------------------------------------------------ responses / anthropic
@dataclass
class ProtocolRequest:
    """Common shape of the Responses and Anthropic Messages profiles after parsing."""
    model: str
    messages: list
    system: str
    chain: S.SamplerChainConfig
    max_tokens: int
    stream: bool
    stop: tuple
    tools: list
    tool_choice: object
    parallel_tool_calls: bool
    metadata: dict
    resumable: bool
    thinking: bool
    tool_history: list = field(default_factory=list)


def parse_responses_request(obj) -> ProtocolRequest:
    from ..frontend import tools as T
    _require_obj(obj, "body")
    _check_fields(obj, {"model", "input", "instructions", "max_output_tokens", "temperature", "top_p", "stream",
                        "metadata", "store", "tools", "tool_choice", "parallel_tool_calls", "reasoning", "sllm"},
                  {"previous_response_id", "include", "background", "truncation", "user", "text", "conversation",
                   "prompt", "service_tier", "safety_identifier", "prompt_cache_key", "max_tool_calls", "top_logprobs"})
    if obj.get("store") not in (None, False):
        raise E.unsupported("store: true is not supported", "store")
    inp = obj.get("input")
    system_parts, messages = [], []
    if isinstance(obj.get("instructions"), str):
        system_parts.append(obj["instructions"])
    elif obj.get("instructions") is not None:
        raise E.invalid_value("instructions must be a string", "instructions")
    if isinstance(inp, str):
        if not inp:
            raise E.invalid_value("input must not be empty", "input")
        messages.append(ChatMessage("user", inp))
    elif isinstance(inp, list) and inp:
        seen_ordinary = False
        for i, item in enumerate(inp):
            _require_obj(item, f"input[{i}]")
            typ = item.get("type", "message")
            if typ == "message":
                _check_fields(item, {"type", "role", "content", "id", "status"}, prefix=f"input[{i}].")
                role = item.get("role")
                content = item.get("content")
                if isinstance(content, list):
                    texts = []
                    for part in content:
                        if not isinstance(part, dict) or part.get("type") not in ("input_text", "output_text", "text") \
                                or not isinstance(part.get("text"), str):
                            raise E.unsupported("only text content parts are supported", f"input[{i}].content")
                        texts.append(part["text"])
                    content = "".join(texts)
                if not isinstance(content, str):
                    raise E.invalid_value("message content must be text", f"input[{i}].content")
                if role in ("system", "developer"):
                    if seen_ordinary:
                        raise E.invalid_value("system / developer items must precede ordinary messages", f"input[{i}]")
                    system_parts.append(content)
                elif role in ("user", "assistant"):
                    seen_ordinary = True
                    messages.append(ChatMessage(role, content))
                else:
                    raise E.invalid_value("unsupported role", f"input[{i}].role")
            elif typ == "function_call":
                _check_fields(item, {"type", "call_id", "name", "arguments", "id", "status"}, prefix=f"input[{i}].")
                seen_ordinary = True
                messages.append(ChatMessage("assistant", '{"tool_calls":[{"name":%s,"arguments":%s}]}' % (
                    __import__("json").dumps(item.get("name")), item.get("arguments") or "{}")))
            elif typ == "function_call_output":
                _check_fields(item, {"type", "call_id", "output", "id", "status"}, prefix=f"input[{i}].")
                if not isinstance(item.get("call_id"), str) or len(item["call_id"]) > 256 or not isinstance(item.get("output"), str):
                    raise E.invalid_value("function_call_output needs call_id and string output", f"input[{i}]")
                seen_ordinary = True
                messages.append(ChatMessage("user", T.render_tool_result(item["call_id"], item["output"])))
            else:
                raise E.unsupported(f"input item type {typ} is not supported", f"input[{i}].type")
    else:
        raise E.invalid_value("input must be a string or a non-empty array", "input")
    if not any(m.role == "user" for m in messages):
        raise E.invalid_value("at least one user message is required", "input")
    tools, choice = [], None
    if obj.get("tools") is not None:
        raw = obj["tools"]
        if not isinstance(raw, list) or len(raw) > 128:
            raise E.invalid_value("tools must be an array of at most 128 functions", "tools")
        norm = []
        for t in raw:
            if not isinstance(t, dict) or t.get("type") != "function":
                raise E.unsupported("only client function tools are supported", "tools")
            _check_fields(t, {"type", "name", "description", "parameters", "strict"}, prefix="tools.")
            norm.append({"type": "function", "function": {k: t[k] for k in ("name", "description", "parameters") if k in t}})
        try:
            tools = T.parse_tools(norm) if norm else []
            tc = obj.get("tool_choice")
            if isinstance(tc, dict) and tc.get("type") == "function" and "name" in tc:
                tc = {"type": "function", "function": {"name": tc["name"]}}
            choice = T.parse_tool_choice(tc, tools) if tools else None
        except T.ToolProtocolError as exc:
            raise E.invalid_value(str(exc), "tools") from None
    elif obj.get("tool_choice") not in (None, "none", "auto"):
        raise E.invalid_value("tool_choice requires tools", "tool_choice")
    md = obj.get("metadata") or {}
    if not isinstance(md, dict) or len(md) > 16 or any(not isinstance(k, str) or len(k) > 64 or not isinstance(v, str) or len(v) > 512 for k, v in md.items()):
        raise E.invalid_value("metadata: at most 16 string pairs (key <= 64, value <= 512)", "metadata")
    thinking = False
    if obj.get("reasoning") is not None:
        r = _require_obj(obj["reasoning"], "reasoning")
        _check_fields(r, {"effort"}, {"summary", "generate_summary"}, prefix="reasoning.")
        if r.get("effort") not in (None, "none", "minimal", "low", "medium", "high"):
            raise E.invalid_value("invalid reasoning.effort", "reasoning.effort")
        thinking = r.get("effort") in ("low", "medium", "high")
    resumable = False
    if obj.get("sllm") is not None:
        ext = _require_obj(obj["sllm"], "sllm")
        _check_fields(ext, {"resumable"}, prefix="sllm.")
        resumable = _bool(ext, "resumable")
    max_tokens = _int_in(obj, "max_output_tokens", 1, MAX_COMPLETION_TOKENS, 256)
    stream = _bool(obj, "stream")
    if resumable and (not stream or max_tokens > 40):
        raise E.invalid_value("sllm.resumable requires stream: true and max_output_tokens <= 40", "sllm.resumable")
    chain = _common_sampling(obj, "max_output_tokens")
    return ProtocolRequest(_model(obj), messages, "\n\n".join(system_parts), chain, max_tokens, stream, (), tools, choice,
                           _bool(obj, "parallel_tool_calls", True), md, resumable, thinking)


def parse_anthropic_request(obj) -> ProtocolRequest:
    from ..frontend import tools as T
    import json
    _require_obj(obj, "body")
    _check_fields(obj, {"model", "messages", "system", "max_tokens", "temperature", "top_p", "top_k", "stream",
                        "stop_sequences", "metadata", "tools", "tool_choice", "sllm"},
                  {"thinking", "service_tier", "container", "mcp_servers", "context_management"})
    if "max_tokens" not in obj:
        raise E.invalid_value("max_tokens is required", "max_tokens")
    system = obj.get("system", "")
    if isinstance(system, list):
        parts = []
        for b in system:
            if not isinstance(b, dict) or b.get("type") != "text" or not isinstance(b.get("text"), str):
                raise E.unsupported("system blocks must be text", "system")
            parts.append(b["text"])
        system = "\n\n".join(parts)
    if not isinstance(system, str):
        raise E.invalid_value("system must be a string or text blocks", "system")
    raw = obj.get("messages")
    if not isinstance(raw, list) or not raw or len(raw) > MAX_MESSAGES:
        raise E.invalid_value("messages must be a non-empty array", "messages")
    messages = []
    for i, m in enumerate(raw):
        _require_obj(m, f"messages[{i}]")
        _check_fields(m, {"role", "content"}, prefix=f"messages[{i}].")
        role = m.get("role")
        if role not in ("user", "assistant"):
            raise E.invalid_value("role must be user or assistant", f"messages[{i}].role")
        c = m.get("content")
        if isinstance(c, str):
            messages.append(ChatMessage(role, c))
            continue
        if not isinstance(c, list) or not c:
            raise E.invalid_value("content must be a string or a non-empty block array", f"messages[{i}].content")
        texts = []
        for b in c:
            if not isinstance(b, dict):
                raise E.invalid_value("content blocks must be objects", f"messages[{i}].content")
            bt = b.get("type")
            if bt == "text" and isinstance(b.get("text"), str):
                texts.append(b["text"])
            elif bt == "tool_use" and role == "assistant":
                texts.append(json.dumps({"tool_calls": [{"name": b.get("name"), "arguments": b.get("input") or {}}]}))
            elif bt == "tool_result" and role == "user":
                content = b.get("content")
                if isinstance(content, list):
                    content = "".join(x.get("text", "") for x in content if isinstance(x, dict) and x.get("type") == "text")
                if not isinstance(content, str) or not isinstance(b.get("tool_use_id"), str):
                    raise E.invalid_value("tool_result needs tool_use_id and text content", f"messages[{i}].content")
                texts.append(T.render_tool_result(b["tool_use_id"], content))
            else:
                raise E.unsupported(f"content block type {bt} is not supported", f"messages[{i}].content")
        messages.append(ChatMessage(role, "".join(texts)))
    if messages[0].role != "user":
        raise E.invalid_value("the first message must be from the user", "messages")
    tools, choice = [], None
    if obj.get("tools") is not None:
        if not isinstance(obj["tools"], list) or len(obj["tools"]) > 128:
            raise E.invalid_value("tools must be an array of at most 128 entries", "tools")
        norm = []
        for t in obj["tools"]:
            if not isinstance(t, dict) or t.get("type", "custom") not in ("custom",):
                raise E.unsupported("only client tools are supported", "tools")
            _check_fields(t, {"type", "name", "description", "input_schema"}, {"cache_control"}, prefix="tools.")
            norm.append({"type": "function", "function": {"name": t.get("name"), "description": t.get("description", ""),
                                                          "parameters": t.get("input_schema")}})
        try:
            tools = T.parse_tools(norm) if norm else []
            tc = obj.get("tool_choice")
            if isinstance(tc, dict):
                _check_fields(tc, {"type", "name", "disable_parallel_tool_use"}, prefix="tool_choice.")
                kind = tc.get("type")
                tc = {"auto": "auto", "any": "required", "none": "none"}.get(kind) or \
                    ({"type": "function", "function": {"name": tc.get("name")}} if kind == "tool" else "invalid")
            choice = T.parse_tool_choice(tc, tools) if tools else None
        except T.ToolProtocolError as exc:
            raise E.invalid_value(str(exc), "tools") from None
    chain = _common_sampling(obj, "max_tokens")
    tk = _int_in(obj, "top_k", 1, 1_000_000, None)
    chain.top_k = tk
    stops = obj.get("stop_sequences")
    stop = ()
    if stops is not None:
        if not isinstance(stops, list) or not 1 <= len(stops) <= MAX_STOP or any(not isinstance(s, str) or not s for s in stops) \
                or len(set(stops)) != len(stops):
            raise E.invalid_value("stop_sequences must hold 1-4 unique non-empty strings", "stop_sequences")
        stop = tuple(stops)
    md = obj.get("metadata") or {}
    if not isinstance(md, dict) or set(md) - {"user_id"}:
        raise E.invalid_value("metadata supports only user_id", "metadata")
    resumable = False
    if obj.get("sllm") is not None:
        ext = _require_obj(obj["sllm"], "sllm")
        _check_fields(ext, {"resumable"}, prefix="sllm.")
        resumable = _bool(ext, "resumable")
    return ProtocolRequest(_model(obj), messages, system, chain, _int_in(obj, "max_tokens", 1, MAX_COMPLETION_TOKENS, 256),
                           _bool(obj, "stream"), stop, tools, choice, True, md, resumable, False)

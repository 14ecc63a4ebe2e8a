"""Completions / embeddings / rerank / token utilities / infill / Responses / Anthropic profiles, and the
real engine (CPU tiny model) served over HTTP with continuous batching."""
import base64
import json
import struct
import threading

import numpy as np
import pytest
from fastapi.testclient import TestClient

from sllm_b200.engine.engine import build_engine
from sllm_b200.frontend.text import ByteTokenizer
from sllm_b200.models.config import tiny_llama
from sllm_b200.server.app import ModelRegistry, ServerConfig, build_app
from sllm_b200.server.backend import EngineBackend, ScriptBackend

M = "fixture-model"


def client(backend=None, **cfg):
    backend = backend or ScriptBackend(aliases=(M,))
    return TestClient(build_app(ModelRegistry({M: backend}), ServerConfig(**cfg))), backend


def named_events(resp):
    out, name = [], None
    for line in resp.text.split("\n"):
        if line.startswith("event: "):
            name = line[7:]
        elif line.startswith("data: "):
            out.append((name, json.loads(line[6:])))
    return out


def test_completions_shapes_and_stream():
    c, b = client()
    r = c.post("/v1/completions", json={"model": M, "prompt": "abc", "max_tokens": 4})
    assert r.status_code == 200 and r.json()["object"] == "text_completion" and r.json()["choices"][0]["text"] == "Hello, world"
    r = c.post("/v1/completions", json={"model": M, "prompt": ["a", "b"], "n": 2, "echo": True})
    assert [ch["index"] for ch in r.json()["choices"]] == [0, 1, 2, 3] and r.json()["choices"][2]["text"].startswith("b")
    assert c.post("/v1/completions", json={"model": M, "prompt": [1, 2, 3]}).status_code == 200
    assert c.post("/v1/completions", json={"model": M, "prompt": [[1, 2], [3]]}).status_code == 200
    for bad in ({"model": M, "prompt": []}, {"model": M, "prompt": [1, "a"]}, {"model": M, "prompt": "x", "max_tokens": 0},
                {"model": M, "prompt": "x", "best_of": 2}, {"model": M, "prompt": [999999]}):
        assert c.post("/v1/completions", json=bad).status_code == 400
    r = c.post("/v1/completions", json={"model": M, "prompt": "x", "stream": True})
    lines = [l for l in r.text.split("\n") if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]" and json.loads(lines[0][6:])["choices"][0]["text"] == "Hello"


def test_embeddings_rerank_and_utilities():
    c, b = client()
    r = c.post("/v1/embeddings", json={"model": M, "input": ["alpha", "beta"]})
    d = r.json()["data"]
    assert [x["index"] for x in d] == [0, 1] and abs(np.linalg.norm(d[0]["embedding"]) - 1) < 1e-5
    r64 = c.post("/v1/embeddings", json={"model": M, "input": "alpha", "encoding_format": "base64"}).json()["data"][0]["embedding"]
    vals = struct.unpack("<8f", base64.b64decode(r64))
    assert np.allclose(vals, d[0]["embedding"], atol=1e-6)
    assert c.post("/v1/embeddings", json={"model": M, "input": "x", "dimensions": 4}).status_code == 400
    assert c.post("/v1/embeddings", json={"model": M, "input": ""}).status_code == 400
    r = c.post("/v1/rerank", json={"model": M, "query": "alpha", "documents": ["zzz", "alpha", "alpha"], "top_n": 2, "return_documents": True})
    res = r.json()["results"]
    assert [x["index"] for x in res] == [1, 2] and res[0]["document"]["text"] == "alpha"   # ties keep input order
    assert c.post("/v1/rerank", json={"model": M, "query": "q", "documents": ["a"], "top_n": 2}).status_code == 400
    t = c.post("/v1/tokenize", json={"model": M, "content": "hé<|im_end|>", "with_pieces": True}).json()
    assert t["count"] == len(t["tokens"]) == 4 and t["tokens"][-1] == 258
    assert c.post("/v1/detokenize", json={"model": M, "tokens": t["tokens"]}).json()["content"] == "hé<|im_end|>"
    assert c.post("/v1/detokenize", json={"model": M, "tokens": [10 ** 7]}).status_code == 400
    msgs = [{"role": "user", "content": "hi"}]
    p = c.post("/v1/apply-template", json={"model": M, "messages": msgs, "thinking": "enabled"}).json()["prompt"]
    assert p == "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n<think>\n"
    n = c.post("/v1/input-tokens", json={"model": M, "messages": msgs}).json()
    assert n["input_tokens"] == len(ByteTokenizer().encode(p.replace("<think>\n", "<think>\n\n</think>\n\n"))) and n["context_length"] == 4096
    r = c.post("/v1/infill", json={"model": M, "input_prefix": "def f(", "input_suffix": "): pass", "max_tokens": 3})
    assert r.status_code == 200 and r.json()["object"] == "infill"
    assert "<|fim_suffix|>" in b.tokenizer.decode(b.submitted[-1][0])


def test_responses_profile():
    c, b = client()
    r = c.post("/v1/responses", json={"model": M, "input": "hello", "instructions": "be brief", "max_output_tokens": 8})
    o = r.json()
    assert r.status_code == 200 and o["object"] == "response" and o["id"].startswith("resp_") and o["status"] == "completed"
    assert o["output_text"] == "Hello, world" and o["output"][0]["content"][0]["type"] == "output_text"
    assert o["usage"]["total_tokens"] == o["usage"]["input_tokens"] + o["usage"]["output_tokens"] and o["created_at"] > 0
    assert "be brief" in b.tokenizer.decode(b.submitted[-1][0])
    r = c.post("/v1/responses", json={"model": M, "input": [{"role": "developer", "content": "sys"}, {"role": "user", "content": [{"type": "input_text", "text": "q"}]}], "stream": True})
    ev = named_events(r)
    names = [n for n, _ in ev]
    assert names[0] == "response.created" and names[-1] == "response.completed" and "response.output_text.delta" in names
    assert "[DONE]" not in r.text
    assert [d["sequence_number"] for _, d in ev] == list(range(len(ev)))
    for bad, param in (({"model": M, "input": "x", "store": True}, "store"), ({"model": M, "input": "x", "previous_response_id": "r"}, "previous_response_id"),
                       ({"model": M, "input": [{"role": "user", "content": "a"}, {"role": "system", "content": "late"}]}, None),
                       ({"model": M, "input": [{"type": "image", "x": 1}]}, None)):
        rr = c.post("/v1/responses", json=bad)
        assert rr.status_code == 400 and (param is None or rr.json()["error"]["param"] == param)
    # function tools: the scripted model answers with the canonical envelope
    tool = {"type": "function", "name": "get_weather", "description": "w", "parameters": {"type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"], "additionalProperties": False}}
    tb = ScriptBackend(deltas=['{"tool_calls":[{"name":"get_weather",', '"arguments":{"city":"Paris"}}]}'], aliases=(M,))
    c2, _ = client(tb)
    o = c2.post("/v1/responses", json={"model": M, "input": "weather?", "tools": [tool], "tool_choice": "required"}).json()
    fc = o["output"][0]
    assert fc["type"] == "function_call" and fc["name"] == "get_weather" and json.loads(fc["arguments"]) == {"city": "Paris"}
    assert tb.submitted[-1][1].grammar_gbnf and "get_weather" in tb.tokenizer.decode(tb.submitted[-1][0])
    ev = named_events(c2.post("/v1/responses", json={"model": M, "input": "weather?", "tools": [tool], "stream": True}))
    assert "response.function_call_arguments.done" in [n for n, _ in ev]


def test_anthropic_messages_profile():
    c, b = client()
    H = {"anthropic-version": "2023-06-01"}
    body = {"model": M, "max_tokens": 16, "system": "sys", "messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}]}
    o = c.post("/v1/messages", json=body, headers=H).json()
    assert o["type"] == "message" and o["role"] == "assistant" and o["content"] == [{"type": "text", "text": "Hello, world"}]
    assert o["stop_reason"] == "end_turn" and o["usage"]["output_tokens"] == 3
    assert c.post("/v1/messages", json=body).status_code == 400                  # version header is mandatory
    bad = c.post("/v1/messages", json={**body, "thinking": {"type": "enabled"}}, headers=H)
    assert bad.status_code == 400 and bad.json()["type"] == "error" and bad.json()["error"]["type"] == "invalid_request_error"
    assert c.post("/v1/messages", json={k: v for k, v in body.items() if k != "max_tokens"}, headers=H).status_code == 400
    assert c.post("/v1/messages", json={**body, "model": "nope"}, headers=H).json()["error"]["type"] == "not_found_error"
    ev = named_events(c.post("/v1/messages", json={**body, "stream": True}, headers=H))
    names = [n for n, _ in ev]
    assert names[0] == "message_start" and names[-1] == "message_stop" and names.count("content_block_delta") == 3
    assert [n for n in names if n in ("content_block_start", "content_block_stop", "message_delta")] == ["content_block_start", "content_block_stop", "message_delta"]
    tool = {"name": "lookup", "description": "d", "input_schema": {"type": "object", "properties": {"q": {"type": "string"}}, "required": ["q"], "additionalProperties": False}}
    tb = ScriptBackend(deltas=['{"tool_calls":[{"name":"lookup","arguments":{"q":"x"}}]}'], aliases=(M,))
    c2, _ = client(tb)
    o = c2.post("/v1/messages", json={**body, "tools": [tool], "tool_choice": {"type": "any"}}, headers=H).json()
    assert o["stop_reason"] == "tool_use" and o["content"][0]["type"] == "tool_use" and o["content"][0]["input"] == {"q": "x"}


@pytest.fixture(scope="module")
def engine_client():
    cfg = tiny_llama()
    cfg.max_context = 160
    cfg.vocab = 1024
    eng = build_engine(cfg, "cpu", seed=0, max_batch=4, use_cuda_graphs=False)
    backend = EngineBackend(eng, ByteTokenizer(1024), aliases=(M,), queue_capacity=16)
    c = TestClient(build_app(ModelRegistry({M: backend}), ServerConfig(metrics=True)))
    yield c, backend
    backend.shutdown(1.0)


def test_engine_served_over_http_greedy_json_and_concurrency(engine_client):
    c, backend = engine_client
    req = {"model": M, "messages": [{"role": "user", "content": "hello"}], "max_completion_tokens": 12, "temperature": 0}
    a = c.post("/v1/chat/completions", json=req).json()
    b = c.post("/v1/chat/completions", json=req).json()
    assert a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]     # greedy is deterministic
    assert a["usage"]["completion_tokens"] <= 12 and a["choices"][0]["finish_reason"] in ("stop", "length")
    # grammar-constrained output parses as JSON even from a random-weight model
    j = c.post("/v1/chat/completions", json={"model": M, "messages": [{"role": "user", "content": "reply in JSON"}],
                                             "max_completion_tokens": 96, "temperature": 0.9, "seed": 7,
                                             "response_format": {"type": "json_schema", "json_schema": {"name": "t", "schema": {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"}}, "required": ["ok", "n"], "additionalProperties": False}}}}).json()
    ch = j["choices"][0]
    if ch["finish_reason"] == "stop":
        parsed = json.loads(ch["message"]["content"])
        assert set(parsed) == {"ok", "n"} and isinstance(parsed["ok"], bool)
    # seeded sampling reproduces; n > 1 derives distinct streams
    s = {"model": M, "messages": [{"role": "user", "content": "x"}], "max_completion_tokens": 10, "temperature": 1.3, "seed": 5, "n": 2}
    r1, r2 = c.post("/v1/chat/completions", json=s).json(), c.post("/v1/chat/completions", json=s).json()
    assert [x["message"]["content"] for x in r1["choices"]] == [x["message"]["content"] for x in r2["choices"]]
    # concurrent requests share decode rounds (continuous batching)
    before = backend.loop.rounds["decode"]
    outs = []
    ts = [threading.Thread(target=lambda: outs.append(c.post("/v1/chat/completions", json=req).json())) for _ in range(4)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert len(outs) == 4 and all(o["choices"][0]["message"]["content"] == a["choices"][0]["message"]["content"] for o in outs)
    assert backend.loop.rounds["decode"] - before < 4 * 12
    e = c.post("/v1/embeddings", json={"model": M, "input": ["abc", "abd"]}).json()["data"]
    assert len(e[0]["embedding"]) == 256 and abs(np.linalg.norm(e[0]["embedding"]) - 1) < 1e-4
    assert "sllm_tokens_total" in c.get("/metrics").text
    # every finished request left an audit record: what it asked for, what it cost, how it ended
    audit = c.get("/props").json()["request_audit"][M]
    assert audit and audit[-1]["finish_reason"] in ("stop", "length") and audit[-1]["prompt_tokens"] > 0
    assert audit[-1]["total_ms"] >= (audit[-1]["queue_to_first_token_ms"] or 0) and "generated" in audit[-1]
    assert any(r["sampled"] for r in audit) and any(r["constrained"] for r in audit)
    assert c.post("/v1/chat/completions", json={**req, "max_completion_tokens": 4096}).status_code == 400   # context bound


@pytest.mark.parametrize("artifact", ["tiny-shared-moe", "tiny-qwen35", "tiny-qwen35-moe"])
def test_other_model_families_served_from_converted_files(tmp_path, artifact):
    """A mixture-of-experts file and a hybrid (gated delta net) file go convert -> verify -> open_model -> HTTP."""
    import argparse
    from sllm_b200.cli import convert
    from sllm_b200.cli.common import open_model
    g, l = str(tmp_path / "m.gguf"), str(tmp_path / "m.lock.json")
    assert convert.main(["--kind", "random-llama", "--artifact", artifact, "--weight-format", "fp32", "--output", g,
                         "--derived-lock", l, "--synthetic-tokenizer"]) == 0
    args = argparse.Namespace(gguf=g, derived_lock=l, device_index=0, target="sm_100a", kv_cache_encoding=None,
                              context_length=None, cpu=True)
    eng, tok, _, _ = open_model(args, max_batch=2)
    backend = EngineBackend(eng, tok, aliases=(M,), queue_capacity=4)
    try:
        c = TestClient(build_app(ModelRegistry({M: backend}), ServerConfig()))
        req = {"model": M, "prompt": "alpha beta gamma", "max_tokens": 6, "temperature": 0}
        a, b = c.post("/v1/completions", json=req).json(), c.post("/v1/completions", json=req).json()
        assert a["choices"][0]["text"] == b["choices"][0]["text"] and a["usage"]["completion_tokens"] == 6
        props = c.get("/props").json()["models"][0]
        assert props["model_family"] == eng.cfg.family and props["quarantine"] is None
    finally:
        backend.shutdown(1.0)


def test_activation_encoding_flag_serves_the_w4a4_path(tmp_path):
    """`--activation-encoding fp4`: a mixture-of-experts file served with 4-bit activations (CPU form of the W4A4
    arithmetic); /props reports it and greedy completions are reproducible."""
    import argparse
    from sllm_b200.cli import convert
    from sllm_b200.cli.common import open_model
    from sllm_b200.ops import w4
    g, l = str(tmp_path / "m.gguf"), str(tmp_path / "m.lock.json")
    assert convert.main(["--kind", "random-llama", "--artifact", "tiny-shared-moe", "--weight-format", "bf16", "--output", g,
                         "--derived-lock", l, "--synthetic-tokenizer"]) == 0
    args = argparse.Namespace(gguf=g, derived_lock=l, device_index=0, target="sm_100a", kv_cache_encoding=None,
                              context_length=None, cpu=True, activation_encoding="fp4")
    try:
        eng, tok, _, _ = open_model(args, max_batch=2)
        assert w4.w4a4_enabled()
        backend = EngineBackend(eng, tok, aliases=(M,), queue_capacity=4)
        try:
            c = TestClient(build_app(ModelRegistry({M: backend}), ServerConfig()))
            req = {"model": M, "prompt": "alpha beta gamma", "max_tokens": 5, "temperature": 0}
            a, b = c.post("/v1/completions", json=req).json(), c.post("/v1/completions", json=req).json()
            assert a["choices"][0]["text"] == b["choices"][0]["text"] and a["usage"]["completion_tokens"] == 5
            assert c.get("/props").json()["models"][0]["activation_encoding"] == "fp4"
        finally:
            backend.shutdown(1.0)
    finally:
        w4.set_w4a4(False)

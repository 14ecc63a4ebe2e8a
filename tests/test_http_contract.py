"""HTTP contract with scripted backends (no GPU): routes, strict validation, status / code matrix, SSE
framing, disconnect / timeout / 429 / mid-stream error, auth, metrics, replay, admin routes."""
import json
import threading
import time

import pytest
from fastapi.testclient import TestClient

from sllm_b200.server.app import ModelRegistry, ServerConfig, build_app
from sllm_b200.server.backend import BlockingBackend, EndlessBackend, FailOnceBackend, ScriptBackend
from sllm_b200.server.lifecycle import ServerLifecycle
from sllm_b200.server.security import CredentialStore

MODEL = "fixture-model"
HELLO = {"model": MODEL, "messages": [{"role": "user", "content": "hello"}]}


def client(backend=None, **cfg):
    backend = backend or ScriptBackend(aliases=(MODEL,))
    app = build_app(ModelRegistry({MODEL: backend}), ServerConfig(**cfg))
    return TestClient(app), backend


def sse_events(resp):
    return [l[6:] for l in resp.text.split("\n") if l.startswith("data: ")]


def test_valid_requests_and_response_shape():
    c, b = client()
    r = c.post("/v1/chat/completions", json=HELLO)
    assert r.status_code == 200
    body = r.json()
    assert body["object"] == "chat.completion" and body["model"] == MODEL and body["id"].startswith("chatcmpl-")
    ch = body["choices"][0]
    assert ch["index"] == 0 and ch["message"] == {"role": "assistant", "content": "Hello, world"} and ch["finish_reason"] == "stop"
    u = body["usage"]
    assert u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"] and u["completion_tokens"] == 3
    full = {"model": MODEL, "messages": [{"role": "system", "content": "be concise"}, {"role": "user", "content": "hello"},
                                           {"role": "assistant", "content": "hi"}, {"role": "user", "content": "again"}],
            "temperature": 0.0, "top_p": 0.9, "max_completion_tokens": 7, "stop": ["\n"], "presence_penalty": 0.5,
            "frequency_penalty": -0.5, "seed": -41, "n": 2, "logit_bias": {"0": -100, "7": 2.5, "4294967295": 1},
            "logprobs": True, "top_logprobs": 2, "stream": False,
            "response_format": {"type": "json_schema", "json_schema": {"name": "a", "schema": {"type": "object", "properties": {"x": {"type": "integer"}}, "required": ["x"], "additionalProperties": False}}},
            "sllm": {"sampling": {"chain_version": 1, "top_k": 40, "min_p": 0.05, "repeat_penalty": 1.1}}}
    r = c.post("/v1/chat/completions", json=full)
    assert r.status_code == 200 and len(r.json()["choices"]) == 2
    assert r.json()["usage"]["completion_tokens"] == 6          # summed over choices, prompt counted once
    prompt_ids, gcfg = b.submitted[-1]
    assert gcfg.max_new_tokens == 7 and gcfg.grammar_gbnf and gcfg.chain.top_k == 40
    assert b.tokenizer.decode(prompt_ids).endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n")


INVALID = [
    ({"messages": HELLO["messages"]}, 400, "invalid_value", "model"),
    ({"model": MODEL, "messages": []}, 400, "invalid_value", "messages"),
    ({"model": "not-served", "messages": HELLO["messages"]}, 404, "model_not_found", "model"),
    ({**HELLO, "future_field": True}, 400, "unsupported_parameter", "future_field"),
    ({**HELLO, "tools": []}, 400, "unsupported_parameter", "tools"),
    ({"model": MODEL, "messages": [{"role": "developer", "content": "x"}]}, 400, "unsupported_parameter", "messages[0].role"),
    ({"model": MODEL, "messages": [{"role": "user", "content": [{"type": "text", "text": "hello"}]}]}, 400, "unsupported_parameter", "messages[0].content"),
    ({**HELLO, "n": 9}, 400, "invalid_value", "n"),
    ({**HELLO, "response_format": {"type": "json_object"}}, 400, "invalid_value", "response_format"),
    ({**HELLO, "top_logprobs": 1}, 400, "invalid_value", "top_logprobs"),
    ({"model": MODEL, "messages": [{"role": "user", "content": "Return JSON."}], "response_format": {"type": "json_schema", "json_schema": {"name": "answer", "schema": {"type": "string", "pattern": "^[a-z]+$"}}}}, 400, "invalid_value", None),
    ({**HELLO, "sllm": {"sampling": {"mirostat": {"version": 2}, "top_k": 4}}}, 400, "invalid_value", "sllm"),
    ({**HELLO, "temperature": "0.5"}, 400, "invalid_value", "temperature"),
    ({**HELLO, "max_tokens": 5}, 400, "unsupported_parameter", "max_tokens"),
    ({**HELLO, "max_completion_tokens": 4097}, 400, "invalid_value", "max_completion_tokens"),
    ({**HELLO, "stop": ["a", "a"]}, 400, "invalid_value", "stop"),
    ({**HELLO, "sllm": {"unknown": 1}}, 400, "unsupported_parameter", "sllm.unknown"),
    ({**HELLO, "sllm": {"separate_reasoning": True}}, 400, "invalid_value", "sllm.separate_reasoning"),
    ({"model": MODEL, "messages": [{"role": "user", "content": "a"}, {"role": "system", "content": "late"}]}, 400, "invalid_value", "messages"),
    ({**HELLO, "logit_bias": {"1": 101}}, 400, "invalid_value", "logit_bias"),
]


@pytest.mark.parametrize("req,status,code,param", INVALID)
def test_reject_matrix(req, status, code, param):
    c, _ = client()
    r = c.post("/v1/chat/completions", json=req)
    assert r.status_code == status, r.text
    err = r.json()["error"]
    assert err["code"] == code and set(err) == {"message", "type", "param", "code"}
    if param is not None:
        assert err["param"] == param


def test_malformed_json_content_type_and_size():
    c, _ = client()
    r = c.post("/v1/chat/completions", content=b"{not json", headers={"content-type": "application/json"})
    assert r.status_code == 400 and r.json()["error"]["code"] == "invalid_json"
    r = c.post("/v1/chat/completions", content=json.dumps(HELLO), headers={"content-type": "text/plain"})
    assert r.status_code == 400
    r = c.post("/v1/chat/completions", content=b"{}", headers={"content-type": "application/json", "content-length": str(97 * 1024 * 1024)})
    assert r.status_code == 413 and r.json()["error"]["code"] == "request_too_large"
    r = c.post("/v1/chat/completions", content=b'{"model": NaN}', headers={"content-type": "application/json"})
    assert r.status_code == 400 and r.json()["error"]["code"] == "invalid_json"


def test_sse_framing_done_and_reasoning_split():
    c, _ = client(ScriptBackend(deltas=[("", "thinking "), ("", "more"), ("The", ""), (" answer", "")], aliases=(MODEL,)))
    r = c.post("/v1/chat/completions", json={**HELLO, "stream": True, "sllm": {"thinking": "enabled", "separate_reasoning": True}})
    assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
    ev = sse_events(r)
    assert ev[-1] == "[DONE]"
    chunks = [json.loads(e) for e in ev[:-1]]
    assert chunks[0]["choices"][0]["delta"] == {"role": "assistant", "content": ""}
    assert all(ch["object"] == "chat.completion.chunk" for ch in chunks)
    reasoning = "".join(ch["choices"][0]["delta"].get("reasoning_content", "") for ch in chunks)
    content = "".join(ch["choices"][0]["delta"].get("content", "") for ch in chunks)
    assert reasoning == "thinking more" and content == "The answer"
    assert chunks[-1]["choices"][0]["finish_reason"] == "stop" and chunks[-1]["choices"][0]["delta"] == {}


def test_mid_stream_error_closes_without_done_and_next_request_works():
    c, _ = client(FailOnceBackend(aliases=(MODEL,)))
    r = c.post("/v1/chat/completions", json={**HELLO, "stream": True})
    ev = sse_events(r)
    assert ev[-1] != "[DONE]" and "error" in json.loads(ev[-1])
    r = c.post("/v1/chat/completions", json=HELLO)
    assert r.status_code == 200
    c2, _ = client(FailOnceBackend(aliases=(MODEL,)))
    assert c2.post("/v1/chat/completions", json=HELLO).status_code == 500


def test_queue_full_is_429_and_length_finish():
    b = BlockingBackend(aliases=(MODEL,), queue_capacity=1)
    c, _ = client(b)
    results = {}
    t = threading.Thread(target=lambda: results.setdefault("first", c.post("/v1/chat/completions", json=HELLO)))
    t.start()
    for _ in range(200):
        if b.active:
            break
        time.sleep(0.01)
    r = c.post("/v1/chat/completions", json=HELLO)
    assert r.status_code == 429 and r.json()["error"]["code"] == "rate_limit_exceeded" and r.json()["error"]["type"] == "rate_limit_error"
    b.release.set()
    t.join(10)
    assert results["first"].status_code == 200
    c3, _ = client(EndlessBackend(aliases=(MODEL,)))
    r = c3.post("/v1/chat/completions", json={**HELLO, "max_completion_tokens": 5})
    assert r.json()["choices"][0]["finish_reason"] == "length" and r.json()["usage"]["completion_tokens"] == 5


def test_request_timeout_cancels_backend():
    b = BlockingBackend(aliases=(MODEL,))
    c, _ = client(b, request_timeout_s=0.2)
    r = c.post("/v1/chat/completions", json=HELLO)
    assert r.status_code == 504
    for _ in range(200):
        if b.active == 0:
            break
        time.sleep(0.01)
    assert b.active == 0          # the slot was released by cancellation


def test_auth_roles_keys_reload_and_anthropic_header(tmp_path):
    kf = tmp_path / "keys"
    kf.write_text("user:user-token-1\nadmin:admin-token-1\n")
    creds = CredentialStore.from_key_file(str(kf))
    c, _ = client(credentials=creds, metrics=True)
    assert c.get("/healthz").status_code == 200 and c.get("/readyz").status_code == 200
    assert c.get("/v1/models").status_code == 401
    assert c.get("/v1/models", headers={"authorization": "Bearer nope-nope"}).json()["error"]["code"] == "invalid_api_key"
    uh, ah = {"authorization": "Bearer user-token-1"}, {"authorization": "Bearer admin-token-1"}
    assert c.get("/v1/models", headers=uh).json()["data"][0]["id"] == MODEL
    assert c.get("/slots", headers=uh).status_code == 403 and c.get("/slots", headers=ah).json() == {"slots": []}
    assert c.post("/admin/slots/12345/cancel", headers=uh).status_code == 403
    assert c.post("/admin/slots/12345/cancel", headers=ah).status_code == 404
    assert c.get("/metrics", headers=uh).status_code == 200
    kf.write_text("user:user-token-2\nadmin:admin-token-1\n")
    assert c.post("/admin/keys/reload", headers=ah).json()["keys"] == 2
    assert c.get("/v1/models", headers=uh).status_code == 401
    assert c.get("/v1/models", headers={"authorization": "Bearer user-token-2"}).status_code == 200
    r = c.post("/v1/messages", json={"model": MODEL, "max_tokens": 5, "messages": [{"role": "user", "content": "hi"}]},
               headers={"x-api-key": "user-token-2", "anthropic-version": "2023-06-01"})
    assert r.status_code == 200
    r = c.post("/v1/messages", json={"model": MODEL, "max_tokens": 5, "messages": [{"role": "user", "content": "hi"}]},
               headers={"anthropic-version": "2023-06-01"})
    assert r.status_code == 401 and r.json()["type"] == "error" and r.json()["error"]["type"] == "authentication_error"


def test_open_and_legacy_user_key_roles_are_separated():
    """An open store and the single legacy key grant the user surface only; admin needs an explicit admin key."""
    open_store = CredentialStore.open()
    assert open_store.role_for(None) == "user" and not open_store.protected
    legacy = CredentialStore.from_user_key("user-secret")
    assert legacy.role_for("Bearer user-secret") == "user"
    assert legacy.role_for("Bearer other-secret") is None and legacy.role_for("Basic user-secret") is None
    c, _ = client(credentials=legacy)
    h = {"authorization": "Bearer user-secret"}
    assert c.get("/v1/models", headers=h).status_code == 200
    for path in ("/admin/slots/1/cancel", "/admin/keys/reload", f"/admin/models/{MODEL}/unload", "/admin/models/evict-idle"):
        assert c.post(path, headers=h).status_code == 403, path
    c_open, _ = client()
    for path in ("/admin/slots/1/cancel", f"/admin/models/{MODEL}/load", "/admin/models/evict-idle"):
        assert c_open.post(path).status_code == 403, path


def test_metrics_props_slots_and_lifecycle():
    c, b = client(metrics=True)
    c.post("/v1/chat/completions", json=HELLO)
    text = c.get("/metrics").text
    for fam in ("sllm_requests_total", "sllm_tokens_total", "sllm_request_ttft_seconds_bucket", "sllm_cancellations_total",
                "sllm_http_responses_total", "sllm_scheduler_accepting", "sllm_scheduler_active_requests",
                "sllm_scheduler_queue_capacity", "sllm_scheduler_queue_depth", "sllm_scheduler_slots", "sllm_model_ready",
                "sllm_backend_memory_bytes"):
        assert fam in text
    assert 'sllm_requests_total{model="fixture-model",outcome="completed"} 1' in text
    assert "hello" not in text
    p = c.get("/props").json()
    assert p["lifecycle"] == "ready" and p["models"][0]["id"] == MODEL and "features" in p
    assert c.get("/slots").status_code == 403                             # admin surface: closed without an admin key
    assert c.post("/admin/slots/12345/cancel").status_code == 403      # an open store never grants admin
    c2, _ = client()
    assert c2.get("/metrics").status_code == 404          # opt-in
    life = ServerLifecycle()
    app = build_app(ModelRegistry({MODEL: ScriptBackend(aliases=(MODEL,))}), ServerConfig(), life)
    tc = TestClient(app)
    assert tc.get("/readyz").status_code == 503 and tc.post("/v1/chat/completions", json=HELLO).status_code == 503
    life.to("ready")
    assert tc.get("/readyz").status_code == 200
    life.to("draining")
    assert tc.post("/v1/chat/completions", json=HELLO).status_code == 503


def test_resumable_sse_replay():
    c, _ = client(resumable_sse=True)
    r = c.post("/v1/chat/completions", json={**HELLO, "stream": True, "sllm": {"resumable": True}})
    ids = [int(l[4:]) for l in r.text.split("\n") if l.startswith("id: ")]
    assert ids == sorted(ids) and len(ids) >= 3      # role, content (a backlog travels as one chunk), finish
    cid = json.loads(sse_events(r)[0])["id"]
    again = c.get(f"/v1/chat/completions/{cid}/events", headers={"last-event-id": "2"})
    ev = sse_events(again)
    assert ev[-1] == "[DONE]" and len(ev) == len(sse_events(r)) - 2
    assert c.get("/v1/chat/completions/unknown/events").status_code == 404
    c2, _ = client()
    assert c2.post("/v1/chat/completions", json={**HELLO, "stream": True, "sllm": {"resumable": True}}).status_code == 400
    assert c.post("/v1/chat/completions", json={**HELLO, "sllm": {"resumable": True}}).status_code == 400


def test_openwebui_profile_and_cors():
    c, b = client(compatibility_profile="openwebui", cors_origins=("https://ui.example",))
    assert c.post("/v1/chat/completions", json={**HELLO, "max_tokens": 2}).json()["choices"][0]["finish_reason"] == "length"
    assert c.post("/v1/chat/completions", json={**HELLO, "max_tokens": 2, "max_completion_tokens": 2}).status_code == 400
    r = c.post("/v1/chat/completions", json=HELLO, headers={"origin": "https://ui.example"})
    assert r.headers.get("access-control-allow-origin") == "https://ui.example"
    r = c.post("/v1/chat/completions", json=HELLO, headers={"origin": "https://evil.example"})
    assert "access-control-allow-origin" not in r.headers

"""Command-line tools on the CPU oracle path: converter, sllm commands, server binary, model manifest."""
import json
import os
import signal
import socket
import subprocess
import sys
import threading
import time
import urllib.request

import pytest

from sllm_b200.cli import convert, main as sllm
from sllm_b200.server import errors as E
from sllm_b200.server.model_lifecycle import (ManifestEntry, ManifestError, ModelLifecycleRegistry, parse_manifest)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    d = tmp_path_factory.mktemp("model")
    g, l = str(d / "tiny.gguf"), str(d / "tiny.lock.json")
    assert convert.main(["--kind", "random-llama", "--artifact", "tiny-llama", "--weight-format", "fp32", "--output", g,
                         "--derived-lock", l, "--converter-commit", "test"]) == 0
    return g, l


def run(capsys, argv):
    capsys.readouterr()
    rc = sllm.main(argv)
    out = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines() if x.strip()]
    return rc, out


def src(model):
    return ["--gguf", model[0], "--derived-lock", model[1], "--cpu"]


def test_version_doctor_and_usage(capsys):
    rc, out = run(capsys, ["version"])
    assert rc == 0 and out[0]["target"] == "sm_100a"
    rc, out = run(capsys, ["doctor"])
    assert out[0]["host_library"] is True
    rc, out = run(capsys, ["no-such-command"])
    assert rc == 2 and out[0]["event"] == "error"
    rc, out = run(capsys, [])
    assert rc == 2 and len(out[0]["commands"]) == 17
    rc, out = run(capsys, ["version", "--bogus"])
    assert rc == 2


def test_convert_dry_run_and_verify(capsys, model, tmp_path):
    rc = convert.main(["--kind", "random-llama", "--artifact", "tiny-llama", "--output", str(tmp_path / "x.gguf"),
                       "--derived-lock", str(tmp_path / "x.json"), "--dry-run"])
    assert rc == 0 and not (tmp_path / "x.gguf").exists()
    rc, out = run(capsys, ["verify-model", "--gguf", model[0], "--derived-lock", model[1]])
    assert rc == 0 and out[0]["verified"] and out[0]["tensors"] == 21
    bad = tmp_path / "bad.gguf"
    data = bytearray(open(model[0], "rb").read())
    data[-1] ^= 1
    bad.write_bytes(bytes(data))
    rc, out = run(capsys, ["verify-model", "--gguf", str(bad), "--derived-lock", model[1]])
    assert rc == 3 and "verification failed" in out[0]["message"]
    rc, out = run(capsys, ["generate", "--gguf", model[0], "--derived-lock", model[1], "--target", "gfx1100", "--prompt", "x"])
    assert rc == 2 and "unsupported target" in out[0]["message"]


def test_token_utilities(capsys):
    rc, out = run(capsys, ["tokenize", "--text", "hi there", "--pieces"])
    ids = out[0]["tokens"]
    assert rc == 0 and out[0]["count"] == len(ids) == 8 and len(out[0]["pieces"]) == 8
    rc, out = run(capsys, ["detokenize", "--tokens", " ".join(map(str, ids))])
    assert out[0]["text"] == "hi there"
    rc, out = run(capsys, ["render", "--message", "system:be brief", "--prompt", "hello"])
    assert rc == 0 and "<|im_start|>user\nhello<|im_end|>" in out[0]["prompt"] and out[0]["prompt"].endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n")
    rc, out = run(capsys, ["input-tokens", "--prompt", "hello"])
    assert rc == 0 and out[0]["input_tokens"] == len(out[0]["tokens"]) > 5
    rc, out = run(capsys, ["render", "--message", "nobody:hi"])
    assert rc == 2


def test_apply_template_file(capsys, tmp_path):
    t = tmp_path / "t.jinja"
    t.write_text("{% for m in messages %}[{{ m.role }}] {{ m.content }}\n{% endfor %}{{ extra }}")
    rc, out = run(capsys, ["apply-template", "--prompt", "hello", "--chat-template-file", str(t),
                           "--template-kwargs-json", '{"extra": "END"}'])
    assert rc == 0 and out[0]["prompt"] == "[user] hello\nEND" and len(out[0]["template_sha256"]) == 64
    rc, out = run(capsys, ["apply-template", "--prompt", "hello", "--chat-template-file", str(t),
                           "--chat-template-digest", "0" * 64])
    assert rc == 2
    os.symlink(str(t), str(tmp_path / "link.jinja"))
    rc, out = run(capsys, ["apply-template", "--prompt", "x", "--chat-template-file", str(tmp_path / "link.jinja")])
    assert rc == 2 and "regular" in out[0]["message"]


def test_generate_decode_completions_are_consistent(capsys, model):
    rc, out = run(capsys, ["generate", *src(model), "--prompt", "hi", "--max-new-tokens", "6"])
    assert rc == 0 and out[0]["finish_reason"] == "length" and len(out[0]["tokens"]) == 6
    toks = out[0]["tokens"]
    rc, out2 = run(capsys, ["completions", *src(model), "--prompt", "hi", "--max-new-tokens", "6"])
    assert out2[0]["tokens"] == toks
    rc, rin = run(capsys, ["input-tokens", "--prompt", "hi"])
    ids = " ".join(map(str, rin[0]["tokens"]))
    rc, out3 = run(capsys, ["decode", *src(model), "--input-token-ids", ids, "--max-new-tokens", "6"])
    assert out3[0]["output_tokens"] == toks
    rc, out4 = run(capsys, ["generate", *src(model), "--input-token-ids", ids, "--max-new-tokens", "6", "--temperature", "0.8",
                            "--top-p", "0.9", "--seed", "7"])
    rc, out5 = run(capsys, ["generate", *src(model), "--input-token-ids", ids, "--max-new-tokens", "6", "--temperature", "0.8",
                            "--top-p", "0.9", "--seed", "7"])
    assert out4[0]["tokens"] == out5[0]["tokens"]
    rc, out = run(capsys, ["generate", *src(model), "--prompt", "a", "--message", "user:b"])
    assert rc == 2


def test_embeddings_rerank_infill_benchmark(capsys, model):
    rc, out = run(capsys, ["embeddings", *src(model), "--text", "alpha", "--text", "beta"])
    assert rc == 0 and out[0]["dimensions"] == 256 and len(out[0]["embeddings"]) == 2
    n = sum(x * x for x in out[0]["embeddings"][0]) ** 0.5
    assert abs(n - 1) < 1e-3
    rc, out = run(capsys, ["rerank", *src(model), "--query", "alpha", "--document", "alpha", "--document", "zzz", "--top-n", "1"])
    assert rc == 0 and out[0]["results"][0]["index"] == 0
    rc, out = run(capsys, ["infill", *src(model), "--prefix", "def f(", "--suffix", "):", "--max-new-tokens", "3"])
    assert rc == 0 and out[0]["usage"]["completion_tokens"] == 3
    rc, out = run(capsys, ["benchmark", *src(model), "--prompt", "hi", "--max-new-tokens", "4", "--warmups", "1", "--measured", "1",
                           "--case-id", "c1", "--row-id", "r1"])
    assert rc == 0 and len(out) == 2 and out[1]["measured"] and out[0]["schema"] == "engine-performance-direct-v1"
    names = [e["event"] for e in out[1]["timeline"]]
    assert names[0] == "PrefillSubmit" and "FirstToken" in names and names[-2:] == ["Stop", "Cleanup"]


def test_chat_turns_checkpoint_and_prefix_reuse(capsys, model, tmp_path):
    ck = str(tmp_path / "ck")
    rc, out = run(capsys, ["chat", *src(model), "--system", "s", "--prompt", "first question", "--prompt", "second",
                           "--max-new-tokens", "4", "--checkpoint-directory", ck, "--checkpoint-save", "sess"])
    assert rc == 0
    kinds = [e["event"] for e in out]
    assert kinds[0] == "session_started" and kinds.count("turn_committed") == 2 and "checkpoint_saved" in kinds
    commits = [e for e in out if e["event"] == "turn_committed"]
    assert commits[0]["prefix_hit_tokens"] == 0 and commits[1]["prefix_hit_tokens"] >= 16
    assert all(e["v"] == 1 for e in out)
    rc, out = run(capsys, ["chat", *src(model), "--prompt", "third", "--max-new-tokens", "3", "--checkpoint-directory", ck,
                           "--checkpoint-load", "sess"])
    assert rc == 0
    loaded = [e for e in out if e["event"] == "checkpoint_loaded"][0]
    assert loaded["messages"] == 5
    assert [e for e in out if e["event"] == "turn_committed"][0]["prefix_hit_tokens"] >= 16
    rc, out = run(capsys, ["chat", *src(model), "--prompt", "x", "--checkpoint-load", "nope", "--checkpoint-directory", ck])
    assert rc == 3


# ------------------------------------------------------------------------------------------ manifest / lifecycle
def test_manifest_parsing(tmp_path):
    ok = {"schema_version": "sllm-model-manifest-v1", "models": [
        {"alias": "a", "gguf": "a.gguf", "derived_lock": "a.json", "preload": True, "context_length": 4096},
        {"alias": "b", "gguf": "/abs/b.gguf", "derived_lock": "b.json", "kv_cache_encoding": "fp8"}]}
    es = parse_manifest(json.dumps(ok).encode(), "/base")
    assert es[0].gguf == "/base/a.gguf" and es[1].gguf == "/abs/b.gguf" and es[0].preload and es[1].kv_cache_encoding == "fp8"
    for mut in (lambda d: d.update(extra=1), lambda d: d.update(schema_version="v2"), lambda d: d["models"].append(d["models"][0]),
                lambda d: d["models"][0].update(unknown=1), lambda d: d["models"][0].update(kv_cache_encoding="int4"),
                lambda d: d["models"][0].update(alias="a/b"), lambda d: d.update(models=[])):
        bad = json.loads(json.dumps(ok))
        mut(bad)
        with pytest.raises(ManifestError):
            parse_manifest(json.dumps(bad).encode())


class FakeBackend:
    def __init__(self, alias):
        self.alias, self.closed = alias, False

    def shutdown(self, *a):
        self.closed = True


def test_lifecycle_registry_coalesces_evicts_and_quarantines():
    entries = [ManifestEntry(a, a + ".gguf", a + ".json") for a in ("a", "b", "c", "bad")]
    loads, gate = [], threading.Event()

    def loader(e):
        loads.append(e.alias)
        if e.alias == "bad":
            raise RuntimeError("corrupt")
        if e.alias == "a":
            gate.wait(2.0)
        return FakeBackend(e.alias)

    reg = ModelLifecycleRegistry(entries, loader, max_resident=2)
    got = []
    ts = [threading.Thread(target=lambda: got.append(reg.acquire("a"))) for _ in range(4)]
    for t in ts:
        t.start()
    time.sleep(0.1)
    assert reg.states()["a"]["state"] == "loading"
    gate.set()
    for t in ts:
        t.join()
    assert loads.count("a") == 1 and len(got) == 4 and reg.states()["a"]["leases"] == 4
    b, lease_b = reg.acquire("b")
    with pytest.raises(E.ApiError) as ei:            # both resident models are leased: no capacity for a third
        reg.acquire("c")
    assert ei.value.status == 503
    for _, l in got:
        l.release()
    c, lease_c = reg.acquire("c")                    # evicts idle "a" (least recently used, unleased)
    st = reg.states()
    assert st["a"]["state"] == "unloaded" and st["b"]["state"] == "ready" and got[0][0].closed
    lease_b.release(); lease_c.release()
    with pytest.raises(E.ApiError):
        reg.acquire("bad")
    assert reg.states()["bad"]["state"] == "quarantined"
    with pytest.raises(E.ApiError) as ei:
        reg.acquire("bad")
    assert ei.value.code == "model_quarantined" and loads.count("bad") == 1
    assert reg.admin("bad", "clear-quarantine") == "unloaded"
    assert reg.admin("b", "unload") == "unloaded" and b.closed
    assert sorted(reg.evict_idle()) == ["c"]
    assert reg.admin("c", "load") == "ready"
    with pytest.raises(E.ApiError):
        reg.acquire("nope")
    reg.shutdown()


# ------------------------------------------------------------------------------------------ server binary
def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _post(url, body, key=None):
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    if key:
        req.add_header("Authorization", "Bearer " + key)
    with urllib.request.urlopen(req, timeout=60) as r:
        return json.loads(r.read())


@pytest.mark.timeout(180)
def test_server_binary_ready_serve_and_shutdown_audit(model, tmp_path):
    port = _free_port()
    manifest = tmp_path / "models.json"
    manifest.write_text(json.dumps({"schema_version": "sllm-model-manifest-v1", "models": [
        {"alias": "tiny", "gguf": model[0], "derived_lock": model[1], "preload": False, "max_batch": 4}]}))
    keys = tmp_path / "keys"
    keys.write_text("user:" + "k" * 32 + "\nadmin:" + "a" * 32 + "\n")
    env = dict(os.environ, SLLM_TEST_KEY="k" * 32, SLLM_TEST_ADMIN_KEY="a" * 32, PYTHONPATH=ROOT)
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "sllm-server"), "--models", str(manifest), "--cpu",
                             "--listen", f"127.0.0.1:{port}", "--api-key-file", str(keys), "--metrics", "--prefix-cache",
                             "--max-batch", "4", "--shutdown-timeout-seconds", "5"],
                            stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
    try:
        ready = json.loads(proc.stdout.readline())
        assert ready["event"] == "ready" and ready["models"] == ["tiny"] and ready["authenticated"] and ready["dynamic_models"]
        base = f"http://127.0.0.1:{port}"
        with pytest.raises(urllib.error.HTTPError) as ei:
            _post(base + "/v1/chat/completions", {"model": "tiny", "messages": [{"role": "user", "content": "hi"}]})
        assert ei.value.code == 401
        r = _post(base + "/v1/chat/completions", {"model": "tiny", "messages": [{"role": "user", "content": "hi"}],
                                                   "max_completion_tokens": 4}, "k" * 32)
        assert r["usage"]["completion_tokens"] == 4 and r["choices"][0]["finish_reason"] == "length"
        rc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "sllm"), "models", "list", "--server", base,
                             "--api-key-env", "SLLM_TEST_KEY"], capture_output=True, text=True, env=env)
        assert rc.returncode == 0 and "tiny" in rc.stdout
        # a user key cannot administer models; the admin key can
        rc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "sllm"), "models", "unload", "tiny", "--server", base,
                             "--api-key-env", "SLLM_TEST_KEY"], capture_output=True, text=True, env=env)
        assert rc.returncode == 1
        rc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "sllm"), "models", "unload", "tiny", "--server", base,
                             "--api-key-env", "SLLM_TEST_ADMIN_KEY"], capture_output=True, text=True, env=env)
        assert rc.returncode == 0 and json.loads(rc.stdout)["state"] == "unloaded"
        rc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "sllm"), "models", "list", "--server",
                             "http://example.com:80"], capture_output=True, text=True, env=env)
        assert rc.returncode == 2 and "loopback" in rc.stdout
        proc.send_signal(signal.SIGTERM)
        out, err = proc.communicate(timeout=60)
        audit = json.loads(out.strip().splitlines()[-1])
        assert audit["event"] == "shutdown_audit" and proc.returncode == 0 and "tiny" in audit["dynamic"]
    finally:
        if proc.poll() is None:
            proc.kill()


def test_server_flag_validation(capsys):
    from sllm_b200.cli import server
    for argv in (["--listen", "127.0.0.1:1"], ["--gguf", "x"], ["--gguf", "x", "--derived-lock", "y", "--models", "m"],
                 ["--models", "m", "--tls-cert", "c"], ["--models", "m", "--draft-width", "9"], ["--models", "m", "--listen", "nope"],
                 ["--models", "m", "--context-policy", "keep-prefix-recent"], ["--models", "m", "--checkpoint"],
                 ["--models", "m", "--no-such-flag"]):
        capsys.readouterr()
        assert server.main(argv) == 2
        assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["event"] == "error"


@pytest.mark.timeout(180)
def test_serve_bench_against_live_server(model):
    from sllm_b200.utils import serve_bench
    port = _free_port()
    env = dict(os.environ, PYTHONPATH=ROOT)
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "sllm-server"), "--gguf", model[0], "--derived-lock", model[1],
                             "--model", "tiny", "--cpu", "--listen", f"127.0.0.1:{port}", "--max-batch", "4", "--queue-capacity", "16",
                             "--shutdown-timeout-seconds", "5"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
    try:
        assert json.loads(proc.stdout.readline())["event"] == "ready"
        import asyncio
        import argparse
        a = argparse.Namespace(url=f"http://127.0.0.1:{port}", model="tiny", requests=6, rate=50.0, concurrency=4, prompt_min=20,
                               prompt_max=60, output_min=4, output_max=8, tokens_per_word=1, byte_tokens=True, api_key_env=None,
                               timeout=120.0, seed=1)
        rep = asyncio.run(serve_bench.run(a))
        assert rep["completed"] == 6 and rep["failed"] == 0 and rep["output_tokens"] >= 20
        assert rep["ttft_ms"]["p50"] > 0 and "p50" in rep["itl_ms"]      # (no interval when a backlog arrived as one chunk)
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            proc.communicate(timeout=60)
        except Exception:
            proc.kill()


@pytest.mark.parametrize("artifact", ["tiny-moe", "tiny-shared-moe", "tiny-qwen35", "tiny-qwen35-moe"])
def test_other_families_convert_and_generate(capsys, tmp_path, artifact):
    """The mixture-of-experts and hybrid families go through the same converter, verification and CLI commands."""
    g, l = str(tmp_path / "m.gguf"), str(tmp_path / "m.lock.json")
    assert convert.main(["--kind", "random-llama", "--artifact", artifact, "--weight-format", "fp32", "--output", g,
                         "--derived-lock", l, "--synthetic-tokenizer"]) == 0
    capsys.readouterr()
    rc, out = run(capsys, ["verify-model", "--gguf", g, "--derived-lock", l])
    assert rc == 0 and out[0]["verified"]
    rc, out = run(capsys, ["decode", "--gguf", g, "--derived-lock", l, "--cpu", "--input-token-ids", "5 6 7 8 9", "--max-new-tokens", "5"])
    assert rc == 0 and len(out[0]["output_tokens"]) == 5
    rc, again = run(capsys, ["decode", "--gguf", g, "--derived-lock", l, "--cpu", "--input-token-ids", "5 6 7 8 9", "--max-new-tokens", "5"])
    assert again[0]["output_tokens"] == out[0]["output_tokens"]
    # block-scaled FP8 projections: the hybrid family takes them, the mixture-of-experts family keeps bf16 attention
    rc = convert.main(["--kind", "random-llama", "--artifact", artifact, "--weight-format", "fp8", "--output", g, "--derived-lock", l])
    assert rc == (0 if "qwen35" in artifact else 2)
    capsys.readouterr()
    if rc == 0:
        rc, out = run(capsys, ["decode", "--gguf", g, "--derived-lock", l, "--cpu", "--input-token-ids", "5 6 7 8 9", "--max-new-tokens", "4"])
        assert rc == 0 and len(out[0]["output_tokens"]) == 4

"""Tensor-parallel paths on 2+ GPUs: fused GEMM+all-reduce vs the NCCL baseline vs fp32 maths."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29611 + world), os.path.join(here, "tp_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and "TP_WORKER_OK" in proc.stdout, proc.stdout[-3000:] + proc.stderr[-3000:]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29711 + world), os.path.join(here, "ep_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and "EP_WORKER_OK" in proc.stdout, proc.stdout[-3000:] + proc.stderr[-3000:]


@pytest.mark.parametrize("world", [2])
def test_multi_rank_server_over_http(world, tmp_path):
    """`sllm-server` under torch.distributed.run: rank 0 serves HTTP, the other rank mirrors the engine (tensor-parallel
    FP8 model); greedy completions are deterministic, streaming works, `/props` reports the layout, shutdown is clean."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import json
    import signal
    import socket
    import time
    import urllib.request
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from sllm_b200.cli import convert
    g, lock = str(tmp_path / "m.gguf"), str(tmp_path / "m.lock.json")
    manifest = tmp_path / "shape.json"
    manifest.write_text(json.dumps({"n_layers": 2, "d_model": 1024, "n_heads": 8, "n_kv_heads": 2, "head_dim": 128, "ffn": 2048,
                                    "vocab": 4096, "max_context": 512}))
    assert convert.main(["--kind", "random-llama", "--artifact", "llama3-8b", "--weight-format", "fp8", "--manifest", str(manifest),
                         "--synthetic-tokenizer", "--output", g, "--derived-lock", lock]) == 0
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, PYTHONPATH=root, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29811 + world), os.path.join(root, "bin", "sllm-server"), "--gguf", g, "--derived-lock", lock,
           "--model", "tp", "--listen", f"127.0.0.1:{port}", "--max-batch", "4", "--shutdown-timeout-seconds", "5"]
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
    try:
        ready = None
        t0 = time.time()
        while time.time() - t0 < 240:
            line = proc.stdout.readline()
            if not line:
                break
            if line.startswith("{") and json.loads(line).get("event") == "ready":
                ready = json.loads(line)
                break
        assert ready is not None, proc.stderr.read()[-3000:] if proc.poll() is not None else "server did not become ready"

        def post(path, body):
            req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=json.dumps(body).encode(),
                                         headers={"Content-Type": "application/json"})
            with urllib.request.urlopen(req, timeout=120) as r:
                return r.read().decode()

        body = {"model": "tp", "prompt": "alpha beta gamma delta", "max_tokens": 12, "temperature": 0}
        a = json.loads(post("/v1/completions", body))
        b = json.loads(post("/v1/completions", body))
        assert a["choices"][0]["text"] == b["choices"][0]["text"] and a["usage"]["completion_tokens"] == 12
        sse = post("/v1/completions", {**body, "stream": True})
        assert sse.rstrip().endswith("data: [DONE]") and sse.count("data: ") >= 3
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/props", timeout=30) as r:
            props = json.loads(r.read())
        assert props["models"][0]["tensor_parallel"] == world and props["models"][0]["quarantine"] is None
        # embeddings run on the engine thread and are mirrored to the follower rank
        emb = json.loads(post("/v1/embeddings", {"model": props["models"][0]["id"] if "id" in props["models"][0] else body["model"],
                                                 "input": ["alpha beta gamma", "delta"]}))
        assert len(emb["data"]) == 2 and abs(sum(x * x for x in emb["data"][0]["embedding"]) - 1.0) < 1e-3
        c = json.loads(post("/v1/completions", body))          # generation still works after the mirrored calls
        assert c["choices"][0]["text"] == a["choices"][0]["text"]
        # (numerical agreement of the sharded model with the single-GPU one is the subject of tp_worker.py; greedy text
        # of a random-weight model is decided by near-ties and is not compared across layouts)
    finally:
        proc.send_signal(signal.SIGINT)
        try:
            out, err = proc.communicate(timeout=90)
        except Exception:
            proc.kill()
            out, err = proc.communicate()
    assert "shutdown_audit" in out, err[-2000:]

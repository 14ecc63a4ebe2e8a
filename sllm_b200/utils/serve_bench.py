"""Load generator for a running `sllm-server`: Poisson arrivals, streamed chat completions, p50/p99 TTFT and
inter-token latency, aggregate output tokens per second.

    python -m sllm_b200.utils.serve_bench --url http://127.0.0.1:8080 --model demo --requests 64 --rate 8 \
        --prompt-min 128 --prompt-max 4096 --output-min 64 --output-max 512 [--api-key-env NAME] [--concurrency 64]

Prompts are seeded random words of the requested token count (the byte tokenizer counts one token per byte, a
Hugging Face tokenizer roughly one per word; the report uses the server's own usage counts).  Timing is wall
clock at the client: TTFT = first content delta after the request was sent; ITL = gaps between later deltas.
The reference publishes single-request TTFT / decode rates from its `sllm benchmark` timeline
(crates/sllm-cli/src/benchmark.rs); it has no concurrent load generator because it serves one request at a time.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import random
import statistics
import time


def _pct(xs, p):
    if not xs:
        return None
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(p / 100.0 * (len(xs) - 1))))]


async def _one(session, url, model, prompt, max_tokens, headers, out, temperature=None):
    body = {"model": model, "messages": [{"role": "user", "content": prompt}], "max_completion_tokens": max_tokens, "stream": True}
    if temperature is not None:
        body["temperature"] = temperature
    t0 = time.perf_counter()
    first, last, gaps, usage, err = None, None, [], None, None
    try:
        async with session.post(url + "/v1/chat/completions", json=body, headers=headers) as r:
            if r.status != 200:
                err = f"http {r.status}"
                await r.read()
            else:
                async for raw in r.content:
                    line = raw.decode("utf-8", "replace").strip()
                    if not line.startswith("data:"):
                        continue
                    data = line[5:].strip()
                    if data == "[DONE]":
                        break
                    ev = json.loads(data)
                    if ev.get("usage"):
                        usage = ev["usage"]
                    ch = ev.get("choices") or []
                    if ch and (ch[0].get("delta", {}).get("content") or ch[0].get("delta", {}).get("reasoning_content")):
                        now = time.perf_counter()
                        if first is None:
                            first = now
                        else:
                            gaps.append(now - last)
                        last = now
    except Exception as exc:      # connection errors count as failed requests
        err = type(exc).__name__
    out.append({"ttft": None if first is None else first - t0, "gaps": gaps, "usage": usage, "error": err,
                "total": time.perf_counter() - t0, "stream": None if first is None or last is None else last - first})


async def run(a) -> dict:
    import aiohttp
    rng = random.Random(a.seed)
    words = ["alpha", "beta", "gamma", "delta", "omega", "sigma", "kappa", "theta", "lambda", "zeta"]
    headers = {}
    if a.api_key_env:
        headers["Authorization"] = "Bearer " + os.environ[a.api_key_env]
    results, tasks = [], []
    sem = asyncio.Semaphore(a.concurrency)
    timeout = aiohttp.ClientTimeout(total=a.timeout)
    async with aiohttp.ClientSession(timeout=timeout) as session:
        async def guarded(prompt, n):
            async with sem:
                await _one(session, a.url, a.model, prompt, n, headers, results, getattr(a, "temperature", None))

        t_start = time.perf_counter()
        for _ in range(a.requests):
            n_in = rng.randint(a.prompt_min, a.prompt_max)
            unit = " ".join(rng.choice(words) for _ in range(max(1, n_in // a.tokens_per_word)))
            prompt = unit[:n_in] if a.byte_tokens else unit
            n_out = rng.randint(a.output_min, a.output_max)
            tasks.append(asyncio.create_task(guarded(prompt, n_out)))
            if a.rate > 0:
                await asyncio.sleep(rng.expovariate(a.rate))
        await asyncio.gather(*tasks)
        wall = time.perf_counter() - t_start
    ok = [r for r in results if r["error"] is None]          # a reply without visible text still completed
    ttft = [r["ttft"] for r in ok if r["ttft"] is not None]
    gaps = [g for r in ok for g in r["gaps"]]
    # time per output token of a request: its streaming time over its tokens after the first (a chunk may carry
    # several tokens when the server coalesces a backlog, so this does not depend on chunking)
    tpot = [r["stream"] / (r["usage"]["completion_tokens"] - 1) for r in ok
            if r.get("stream") and r["usage"] and r["usage"].get("completion_tokens", 0) > 1]
    out_tokens = sum((r["usage"] or {}).get("completion_tokens", len(r["gaps"]) + 1) for r in ok)
    in_tokens = sum((r["usage"] or {}).get("prompt_tokens", 0) for r in ok)
    return {"requests": a.requests, "completed": len(ok), "failed": len(results) - len(ok), "wall_s": round(wall, 3),
            "arrival_rate_per_s": a.rate, "concurrency": a.concurrency,
            "output_tokens": out_tokens, "prompt_tokens": in_tokens, "output_tok_per_s": round(out_tokens / wall, 2) if wall > 0 else None,
            "ttft_ms": {"p50": None if not ttft else round(statistics.median(ttft) * 1e3, 2), "p99": None if not ttft else round(_pct(ttft, 99) * 1e3, 2)},
            "itl_ms": {"p50": None if not gaps else round(statistics.median(gaps) * 1e3, 3), "p99": None if not gaps else round(_pct(gaps, 99) * 1e3, 3)},
            "tpot_ms": {"p50": None if not tpot else round(statistics.median(tpot) * 1e3, 3), "p99": None if not tpot else round(_pct(tpot, 99) * 1e3, 3)},
            "errors": sorted({r["error"] for r in results if r["error"]})}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--model", required=True)
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--rate", type=float, default=8.0, help="Poisson arrival rate per second (0 = all at once)")
    ap.add_argument("--concurrency", type=int, default=64)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=4096)
    ap.add_argument("--output-min", type=int, default=64)
    ap.add_argument("--output-max", type=int, default=512)
    ap.add_argument("--tokens-per-word", type=int, default=1)
    ap.add_argument("--byte-tokens", action="store_true", help="the server uses the byte tokenizer: one token per character")
    ap.add_argument("--api-key-env")
    ap.add_argument("--timeout", type=float, default=600.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--temperature", type=float, default=None, help="sampling temperature sent with every request (0 = greedy)")
    a = ap.parse_args(argv)
    print(json.dumps(asyncio.run(run(a))))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

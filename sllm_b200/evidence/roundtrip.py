"""Model-free round trip through the kernel library, run in a child process under a reaper and a circuit breaker.

    python -m sllm_b200.evidence.roundtrip [--state-dir DIR] [--timeout 120]

The child loads the library and pushes a few tiny, model-free launches through it (bf16 and block-scaled FP8 GEMM,
RMSNorm, gated activation, argmax, paged attention over a 2-page cache), each checked against the fp32 restatement,
then reads the device status word.  The parent is the reaper: a child that does not finish in time is killed by its
exact process id and the trip counts as a failure.  A circuit breaker in `state-dir` (one JSON file) opens after
`threshold` consecutive failures: while it is open the trip is not attempted at all (a supervisor that health-checks a
sick GPU must not keep launching work on it); after `cooldown` seconds one trial is let through (half-open), and a
success closes it.  "No GPU" is neither a success nor a failure.  One JSON line on stdout; exit 0 ok / unavailable,
1 failed or reaped, 3 circuit open.

Reference: the private evidence ABI of the native layer (model-free smoke with a watchdog that reaps a stuck child and
a breaker that stops retrying: native/hip/src/evidence_runtime.cpp).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from typing import Optional

SCHEMA = "sllm-roundtrip-v1"


class CircuitBreaker:
    def __init__(self, state_dir: Optional[str], threshold: int = 3, cooldown: float = 300.0, clock=time.time):
        self.path = os.path.join(state_dir, "roundtrip_breaker.json") if state_dir else None
        self.threshold, self.cooldown, self.clock = threshold, cooldown, clock
        self.state = {"consecutive_failures": 0, "opened_at": None}
        if self.path and os.path.exists(self.path):
            try:
                with open(self.path, "r", encoding="utf-8") as f:
                    loaded = json.load(f)
                if isinstance(loaded, dict) and isinstance(loaded.get("consecutive_failures"), int):
                    self.state.update({k: loaded.get(k) for k in self.state})
            except (OSError, ValueError):
                pass                                   # an unreadable state file is an empty one

    def _save(self) -> None:
        if not self.path:
            return
        os.makedirs(os.path.dirname(self.path), exist_ok=True)
        tmp = self.path + ".tmp"
        with open(tmp, "w", encoding="utf-8") as f:
            json.dump(self.state, f)
        os.replace(tmp, self.path)

    def allow(self) -> str:
        """'closed' (go), 'half-open' (one trial after the cooldown) or 'open' (do not try)."""
        if self.state["opened_at"] is None:
            return "closed"
        return "half-open" if self.clock() - self.state["opened_at"] >= self.cooldown else "open"

    def record(self, ok: Optional[bool]) -> None:
        if ok is None:
            return
        if ok:
            self.state = {"consecutive_failures": 0, "opened_at": None}
        else:
            self.state["consecutive_failures"] += 1
            if self.state["consecutive_failures"] >= self.threshold or self.state["opened_at"] is not None:
                self.state["opened_at"] = self.clock()
        self._save()


def run_child(cmd: list, timeout: float) -> dict:
    """Runs `cmd`, reaps it by pid when it overstays, and returns the child's JSON line (or what went wrong)."""
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        out, err = proc.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        proc.kill()                                     # this exact child, nothing else
        out, err = proc.communicate()
        return {"ok": False, "reaped": True, "seconds": round(time.time() - t0, 3), "pid": proc.pid}
    line = next((x for x in reversed(out.strip().splitlines()) if x.startswith("{")), None)
    if line is None:
        return {"ok": False, "reaped": False, "exit_code": proc.returncode, "stderr_tail": err[-400:]}
    try:
        rep = json.loads(line)
    except ValueError:
        return {"ok": False, "reaped": False, "exit_code": proc.returncode, "stderr_tail": "child printed no JSON"}
    rep.update({"reaped": False, "exit_code": proc.returncode, "seconds": round(time.time() - t0, 3)})
    return rep


def roundtrip(state_dir: Optional[str] = None, timeout: float = 120.0, cmd: Optional[list] = None, threshold: int = 3,
              cooldown: float = 300.0, clock=time.time) -> dict:
    br = CircuitBreaker(state_dir, threshold, cooldown, clock)
    gate = br.allow()
    if gate == "open":
        return {"schema": SCHEMA, "ok": False, "circuit": "open", "attempted": False,
                "consecutive_failures": br.state["consecutive_failures"]}
    rep = run_child(cmd or [sys.executable, "-m", "sllm_b200.evidence.roundtrip", "--child"], timeout)
    ok = None if rep.get("unavailable") else bool(rep.get("ok"))
    br.record(ok)
    rep.update({"schema": SCHEMA, "attempted": True, "circuit": br.allow() if ok is not None else gate,
                "consecutive_failures": br.state["consecutive_failures"]})
    return rep


def _child() -> dict:
    try:
        import torch
    except ImportError:
        return {"ok": False, "unavailable": "torch is not importable"}
    if not torch.cuda.is_available():
        return {"ok": False, "unavailable": "no CUDA device"}
    from .. import ops
    from ..ops import _lib, reference as ref
    from ..ops.core import KVLayer, LinearWeight
    if not _lib.kernels_available():
        return {"ok": False, "unavailable": "the kernel library has not been built"}
    dev = "cuda"
    torch.manual_seed(0)
    checks = {}

    def rel(a, b):
        a, b = a.float().cpu(), b.float().cpu()
        return float((a - b).norm() / (b.norm() + 1e-12))

    x = (torch.randn(8, 256, device=dev) * 0.5).bfloat16()
    w = (torch.randn(128, 256, device=dev) * 0.05).bfloat16()
    checks["gemm_bf16"] = rel(ops.linear(x, LinearWeight("dense", w)), x.float() @ w.float().t())
    lw = LinearWeight.from_dense(w.cpu(), "fp8").to(dev)
    xq = ops.quant_fp8(x)
    checks["gemm_fp8"] = rel(ops.linear(xq, lw), ref.linear_fp8(xq.data.cpu(), xq.scale.cpu(), lw.w.cpu(), lw.scale_t.cpu()))
    g = (1 + 0.1 * torch.randn(256, device=dev)).bfloat16()
    checks["rmsnorm"] = rel(ops.rmsnorm(x, g, 1e-5), ref.rmsnorm(x.cpu(), g.cpu(), 1e-5))
    checks["gated_act"] = rel(ops.gated_act(x, "silu"), ref.gated_act(x.cpu(), "silu"))
    lg = torch.randn(4, 1000, device=dev).bfloat16()
    checks["argmax"] = float((ops.argmax(lg).cpu() != lg.float().argmax(1).cpu().int()).sum())
    kv = KVLayer(torch.randn(2, 2, 16, 64, device=dev).bfloat16(), torch.randn(2, 2, 16, 64, device=dev).bfloat16(), None, None,
                 False, 16)
    table = torch.tensor([[0, 1]], dtype=torch.int32, device=dev)
    seq, lens = torch.zeros(1, dtype=torch.int32, device=dev), torch.tensor([29], dtype=torch.int32, device=dev)
    q = torch.randn(1, 4 * 64, device=dev).bfloat16()
    cpu_kv = KVLayer(kv.k.cpu(), kv.v.cpu(), None, None, False, 16)
    checks["paged_attention"] = rel(ops.paged_attention(q, kv, table, seq, lens, 4, 2, 64),
                                    ops.paged_attention(q.cpu(), cpu_kv, table.cpu(), seq.cpu(), lens.cpu(), 4, 2, 64))
    status = ops.device_status(torch.device(dev))
    ok = status == 0 and all(v < 2e-2 for v in checks.values())
    return {"ok": ok, "checks": {k: round(v, 6) for k, v in checks.items()}, "device_status": status,
            "device": torch.cuda.get_device_name(0), "launches": _lib.LAUNCH_COUNT[0]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m sllm_b200.evidence.roundtrip")
    ap.add_argument("--child", action="store_true", help="run the launches in this process (what the parent starts)")
    ap.add_argument("--state-dir", default=None)
    ap.add_argument("--timeout", type=float, default=120.0)
    ap.add_argument("--threshold", type=int, default=3)
    ap.add_argument("--cooldown", type=float, default=300.0)
    a = ap.parse_args(argv)
    if a.child:
        rep = _child()
        print(json.dumps(rep, sort_keys=True), flush=True)
        return 0 if rep.get("ok") or rep.get("unavailable") else 1
    rep = roundtrip(a.state_dir, a.timeout, threshold=a.threshold, cooldown=a.cooldown)
    print(json.dumps(rep, sort_keys=True), flush=True)
    if rep.get("circuit") == "open" and not rep.get("attempted"):
        return 3
    return 0 if rep.get("ok") or rep.get("unavailable") else 1


if __name__ == "__main__":
    sys.exit(main())

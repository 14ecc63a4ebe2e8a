"""Evidence runners: for every kernel family, ONE report that says whether the op computes the right numbers and how
fast it runs against the measured peaks of the machine.

    python -m sllm_b200.evidence --op gemm-fp8 --size small          # one report on stdout
    python -m sllm_b200.evidence --all --out evidence/               # one file per op

A report (schema ``sllm-evidence-v1``) has: ``op``, ``case`` (shapes), ``executed``; when executed ``correctness``
(max_abs, rel_err, tolerance, passed), ``timing`` (median_us over CUDA-event repetitions after warm-up with an L2 flush
between them, algorithmic bytes / flops, achieved GB/s / TFLOP/s and their fraction of the measured copy bandwidth /
bf16 GEMM rate), ``dispatch`` (the launches the op planned: kernel, grid, split plan, fallback_used) and ``device``.
Without a GPU nothing is computed: the report says ``executed: false`` with the reason (the runners never fall back to
a CPU result).  Exit status: 0 all executed reports passed (or none could execute), 1 a check failed, 2 usage.

Reference: the per-op evidence binaries crates/sllm-hip/src/bin/*-evidence.rs (matmul, rmsnorm, rotary, kv-state,
decode / prefill attention, token selector, moe, linear attention, ...), each a correctness + timing report.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
from pathlib import Path

SCHEMA = "sllm-evidence-v1"


def _peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def unavailable_report(op: str, why: str) -> dict:
    return {"schema": SCHEMA, "op": op, "executed": False, "unavailable": why}


def _time(fn, reps: int = 7, warmup: int = 3) -> float:
    import torch
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(ts)


def _check(got, want, rtol: float, atol_frac: float) -> dict:
    got, want = got.float().cpu(), want.float().cpu()
    diff = (got - want).abs()
    tol = rtol * want.abs() + atol_frac * want.abs().max()
    return {"max_abs": float(diff.max()), "rel_err": float((got - want).norm() / (want.norm() + 1e-12)),
            "tolerance": {"rtol": rtol, "atol_frac_of_max": atol_frac}, "elements_off": int((diff > tol).sum()),
            "passed": bool((diff <= tol).all())}


# ---------------------------------------------------------------------------------------------- cases
# every case returns (run, want, bytes, flops, shapes, tolerances); `run()` returns the tensor to compare
def _gemm(fmt: str):
    def make(size):
        import torch
        from .. import ops
        from ..ops import reference as ref
        from ..ops.core import LinearWeight
        m, n, k = {"small": (32, 1024, 1024), "decode": (32, 4096, 4096), "large": (2048, 4096, 4096)}[size]
        torch.manual_seed(1)
        x = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
        if fmt == "bf16":
            lw = LinearWeight("dense", w)
            return (lambda: ops.linear(x, lw)), x.float() @ w.float().t(), 2 * (m * k + n * k + m * n), 2 * m * n * k, \
                {"m": m, "n": n, "k": k}, (1.2e-2, 2e-3)
        if fmt == "fp8":
            lw = LinearWeight.from_dense(w.cpu(), "fp8").to("cuda")
            xq = ops.quant_fp8(x)
            want = ref.linear_fp8(xq.data.cpu(), xq.scale.cpu(), lw.w.cpu(), lw.scale_t.cpu())
            return (lambda: ops.linear(xq, lw)), want, m * k + n * k + 2 * m * n, 2 * m * n * k, {"m": m, "n": n, "k": k}, (1.2e-2, 2e-3)
        from ..ops.w4 import W4Weight, linear_w4
        w4 = W4Weight.quantize(fmt, w.float().cpu(), "cuda", keep_file=False)
        want = x.float().cpu() @ w4.dequantized().t()
        return (lambda: linear_w4(x, w4)), want, 2 * m * k + n * k // 2 + 2 * m * n, 2 * m * n * k, {"m": m, "n": n, "k": k}, (1.5e-2, 4e-3)
    return make


def _rmsnorm(size):
    import torch
    from .. import ops
    from ..ops import reference as ref
    rows, d = {"small": (32, 1024), "decode": (32, 4096), "large": (4096, 4096)}[size]
    x = torch.randn(rows, d, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    return (lambda: ops.rmsnorm(x, w, 1e-5)), ref.rmsnorm(x.cpu(), w.cpu(), 1e-5), 4 * rows * d, 0, {"rows": rows, "d": d}, (1e-2, 4e-3)


def _gated(size):
    import torch
    from .. import ops
    from ..ops import reference as ref
    rows, f = {"small": (32, 1024), "decode": (32, 14336), "large": (2048, 14336)}[size]
    x = torch.randn(rows, 2 * f, device="cuda").bfloat16()
    return (lambda: ops.gated_act(x, "silu")), ref.gated_act(x.cpu(), "silu"), 6 * rows * f, 0, {"rows": rows, "ffn": f}, (1.2e-2, 4e-3)


def _argmax(size):
    import torch
    from .. import ops
    rows, v = {"small": (8, 4096), "decode": (32, 128256), "large": (256, 128256)}[size]
    x = torch.randn(rows, v, device="cuda").bfloat16()
    return (lambda: ops.argmax(x).float()), x.float().argmax(1).float().cpu(), 2 * rows * v, 0, {"rows": rows, "vocab": v}, (0.0, 0.0)


def _attention(size):
    import torch
    from .. import ops
    from ..ops import reference as ref
    from ..ops.core import KVLayer
    batch, ctx = {"small": (4, 256), "decode": (32, 2048), "large": (64, 4096)}[size]
    hq, hkv, hd, page = 32, 8, 128, 16
    blocks = (ctx + page - 1) // page
    pages = batch * blocks
    torch.manual_seed(2)
    kv = KVLayer(torch.randint(0, 120, (pages, hkv, page, hd), dtype=torch.uint8, device="cuda"),
                 torch.randint(0, 120, (pages, hkv, page, hd), dtype=torch.uint8, device="cuda"),
                 torch.rand(pages, hkv, page, device="cuda") * 0.02 + 0.01, torch.rand(pages, hkv, page, device="cuda") * 0.02 + 0.01,
                 True, page)
    table = torch.randperm(pages, device="cuda").int().view(batch, blocks)
    seq = torch.arange(batch, device="cuda", dtype=torch.int32)
    lens = torch.full((batch,), ctx, device="cuda", dtype=torch.int32)
    q = torch.randn(batch, hq * hd, device="cuda").bfloat16()
    cpu_kv = KVLayer(kv.k.cpu(), kv.v.cpu(), kv.k_scale.cpu(), kv.v_scale.cpu(), True, page)
    want = ops.paged_attention(q.cpu(), cpu_kv, table.cpu(), seq.cpu(), lens.cpu(), hq, hkv, hd) if batch * ctx <= 4 * 256 else None
    byts = 2 * batch * ctx * hkv * (hd + 4)
    return (lambda: ops.paged_attention(q, kv, table, seq, lens, hq, hkv, hd, max_kv=ctx)), want, byts, 4 * batch * hq * ctx * hd, \
        {"batch": batch, "ctx": ctx, "hq": hq, "hkv": hkv, "hd": hd, "kv": "fp8"}, (5e-2, 4e-2)   # Q and P are E4M3 on the tensor cores


def _gemm_w4a4(fmt: str):
    """4-bit weights x 4-bit activations on the block-scaled tensor-core kernel, against an fp32 evaluation of the same
    quantised operands (the quantiser's launch is part of the timed op)."""
    def make(size):
        import torch
        from ..ops import reference as ref
        from ..ops.w4 import W4Weight, act_quant_fp4, linear_w4a4, sf_compact
        m, n, k = {"small": (32, 1024, 1024), "decode": (32, 4096, 4096), "large": (32, 28672, 8192)}[size]
        torch.manual_seed(1)
        x = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
        w4 = W4Weight.quantize_device(fmt, (torch.randn(n, k, device="cuda") * 0.05))
        q = act_quant_fp4(x, fmt)
        want = None
        if n * k <= 4096 * 4096:
            xf = ref.dequant_act_fp4(q[0], sf_compact(q[1].cpu()), q[2], fmt)[:, :k]
            want = xf @ w4.dequantized().t()
        return (lambda: linear_w4a4(x, w4)), want, m * k * 2 + n * k * 9 // 16 + 2 * m * n, 2 * m * n * k, \
            {"m": m, "n": n, "k": k, "activations": fmt}, (1.2e-2, 4e-3)
    return make


def _act_quant(size):
    import torch
    from ..ops import reference as ref
    from ..ops.w4 import act_quant_fp4
    rows, k = {"small": (32, 1024), "decode": (32, 8192), "large": (32, 28672)}[size]
    torch.manual_seed(4)
    x = torch.randn(rows, k, device="cuda").bfloat16()
    want = ref.quant_act_fp4(x.cpu(), "nvfp4")[0]            # the packed codes, byte for byte
    return (lambda: act_quant_fp4(x, "nvfp4")[0]), want, rows * k * (2 + 9 / 16), 0, {"rows": rows, "k": k, "format": "nvfp4"}, (0.0, 0.0)


def _gdn(size):
    import torch
    from ..ops import gdn
    seqs, length = {"small": (2, 24), "decode": (16, 1), "large": (1, 2048)}[size]
    qk_heads, v_heads, hd = 4, 8, 128
    t = seqs * length
    torch.manual_seed(5)
    width = (2 * qk_heads + v_heads) * hd
    qkv = (torch.randn(t, width) * 0.5).bfloat16()
    z = torch.randn(t, v_heads * hd).bfloat16()
    b, a = torch.randn(t, v_heads).bfloat16(), torch.randn(t, v_heads).bfloat16()
    a_log, dt_bias, norm_w = torch.randn(v_heads) * 0.5, (torch.randn(v_heads) * 0.5).bfloat16(), 1.0 + torch.randn(hd) * 0.05
    row_off = torch.arange(0, t + 1, length, dtype=torch.int32)
    slots = torch.arange(seqs, dtype=torch.int32)
    st0 = torch.randn(seqs, v_heads, hd, hd) * 0.1
    want = None
    if t <= 64:
        want = gdn.recurrent(qkv, z, b, a, a_log, dt_bias, norm_w, st0.clone(), row_off, slots, qk_heads, v_heads, hd)
    d = lambda v: v.to("cuda")
    args = [d(v) for v in (qkv, z, b, a, a_log, dt_bias, norm_w)]
    st, ro, sl = st0.to("cuda"), d(row_off), d(slots)

    def run():
        st.copy_(st0)
        return gdn.recurrent(*args, st, ro, sl, qk_heads, v_heads, hd)
    byts = 2 * t * (width + 2 * v_heads * hd) + 8 * seqs * v_heads * hd * hd
    return run, want, byts, 4 * t * v_heads * hd * hd, {"sequences": seqs, "tokens_each": length, "v_heads": v_heads}, (2e-2, 1e-2)


def _moe_route(size):
    import torch
    from ..ops import moe as M
    t, e, k = {"small": (64, 32, 4), "decode": (64, 256, 8), "large": (4096, 256, 8)}[size]
    logits = torch.randn(t, e, device="cuda").bfloat16()
    want = M.route(logits.cpu(), k)[1]
    return (lambda: M.route(logits, k)[1]), want, 2 * t * e, 0, {"tokens": t, "experts": e, "top_k": k}, (1e-4, 1e-5)


OPS = {"gemm-bf16": _gemm("bf16"), "gemm-fp8": _gemm("fp8"), "gemm-nvfp4": _gemm("nvfp4"), "gemm-mxfp4": _gemm("mxfp4"),
       "gemm-w4a4-nvfp4": _gemm_w4a4("nvfp4"), "gemm-w4a4-mxfp4": _gemm_w4a4("mxfp4"), "act-quant-fp4": _act_quant,
       "gated-delta-net": _gdn,
       "rmsnorm": _rmsnorm, "gated-act": _gated, "argmax": _argmax, "paged-attention-fp8": _attention, "moe-route": _moe_route}


def run_op(op: str, size: str = "small") -> dict:
    if op not in OPS:
        raise KeyError(op)
    try:
        import torch
    except ImportError:
        return unavailable_report(op, "torch is not importable")
    if not torch.cuda.is_available():
        return unavailable_report(op, "no CUDA device: the evidence runners never compute on the CPU")
    from ..ops import _lib
    if not _lib.kernels_available():
        return unavailable_report(op, "the kernel library has not been built")
    _lib.audit(True)
    _lib.dispatch_records(clear=True)
    run, want, byts, flops, shapes, (rtol, atol) = OPS[op](size)
    got = run()
    torch.cuda.synchronize()
    dispatch = _lib.dispatch_records(clear=True)
    _lib.audit(False)
    us = _time(run)
    hbm, tf, which = _peaks()
    rep = {"schema": SCHEMA, "op": op, "executed": True, "case": {"size": size, **shapes}, "dispatch": dispatch,
           "correctness": _check(got, want, rtol, atol) if want is not None else {"passed": True, "skipped": "oracle too large for this size"},
           "timing": {"median_us": round(us, 2), "bytes": int(byts), "flops": int(flops),
                      "gbs": round(byts / us / 1e3, 1), "tflops": round(flops / us / 1e6, 2),
                      "frac_of_copy_bandwidth": round(byts / (us * 1e-6) / hbm, 3),
                      "frac_of_bf16_gemm_rate": round(flops / (us * 1e-6) / tf, 3) if flops else None, "peaks": which},
           "device": {"name": torch.cuda.get_device_name(0), "capability": list(torch.cuda.get_device_capability(0)),
                      "device_status": int(__import__("sllm_b200").ops.device_status(torch.device("cuda")))}}
    return rep


def validate_report(rep: dict) -> None:
    """Raises ValueError when a report does not follow the schema."""
    if rep.get("schema") != SCHEMA or not isinstance(rep.get("op"), str) or not isinstance(rep.get("executed"), bool):
        raise ValueError("evidence report: schema / op / executed")
    if not rep["executed"]:
        if not isinstance(rep.get("unavailable"), str):
            raise ValueError("evidence report: an unexecuted report states why")
        return
    for key, fields in (("correctness", ("passed",)), ("timing", ("median_us", "bytes", "flops", "gbs", "peaks")), ("device", ("name",))):
        if not isinstance(rep.get(key), dict) or any(f not in rep[key] for f in fields):
            raise ValueError(f"evidence report: {key}")
    if not isinstance(rep.get("dispatch"), list) or not isinstance(rep.get("case"), dict):
        raise ValueError("evidence report: dispatch / case")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m sllm_b200.evidence")
    ap.add_argument("--op", choices=sorted(OPS))
    ap.add_argument("--all", action="store_true")
    ap.add_argument("--size", choices=("small", "decode", "large"), default="small")
    ap.add_argument("--out", help="directory for one JSON file per op (default: stdout, one line per op)")
    a = ap.parse_args(argv)
    if bool(a.op) == bool(a.all):
        ap.print_usage(sys.stderr)
        return 2
    failed = False
    for op in (sorted(OPS) if a.all else [a.op]):
        rep = run_op(op, a.size)
        validate_report(rep)
        failed = failed or (rep["executed"] and not rep["correctness"]["passed"])
        if a.out:
            os.makedirs(a.out, exist_ok=True)
            with open(os.path.join(a.out, f"{op}.{a.size}.json"), "w", encoding="utf-8") as f:
                json.dump(rep, f, indent=1, sort_keys=True)
        else:
            print(json.dumps(rep, sort_keys=True))
    return 1 if failed else 0

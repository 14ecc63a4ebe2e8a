"""Per-kernel micro-benchmarks with roofline fractions.

    python -m sllm_b200.utils.kernel_bench --op gemm --m 32 --n 4096 --k 4096 [--fp8]
    python -m sllm_b200.utils.kernel_bench --op attention --batch 32 --ctx 2048
    python -m sllm_b200.utils.kernel_bench --op prefill --seqs 4 --len 2048
    python -m sllm_b200.utils.kernel_bench --op decode-gemms --m 32 --graph

Timing follows the usual hygiene: warm-up, an L2 flush (a 256 MB write) before each timed launch, CUDA
events on the launching stream, median of the repetitions.  Fractions are reported against the
measured peaks in MEASURED_PEAKS.json at the repository root when present ("of measured"), else
against 6.65 TB/s and 1.59 PFLOP/s ("of fallback").
"""
from __future__ import annotations

import argparse
import json
import math
import statistics
from pathlib import Path

import torch

from .. import ops
from ..ops import reference as ref
from ..ops.core import KVLayer, LinearWeight


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "of measured"
    return 6.65e12, 1.59e15, "of fallback"


_flush = None


def timed(fn, reps: int = 10, warmup: int = 3, flush: bool = True) -> float:
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        if flush:
            _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    return statistics.median(ts)


def timed_graph(fns, reps: int = 5) -> float:
    """Steady-state time per launch: the callables (same op over distinct buffers that together exceed the
    L2 several times over) are captured back to back in one CUDA graph, as a decode step launches them, and
    the replay is timed with events.  Launch latency and L2 reuse are both out of the picture."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for f in fns:
            f()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3 / len(fns))
    return statistics.median(ts)


def _copies(nbytes: int) -> int:
    return max(4, min(64, (3 * 126 * 1024 * 1024) // max(nbytes, 1) + 1))


def bench_gemm(m, n, k, fp8, reps, graph=False):
    dev = "cuda"
    x = torch.randn(m, k, device=dev).bfloat16()
    w = (torch.randn(n, k, device=dev) * 0.02).bfloat16()
    if fp8:
        wq = ops.quant_fp8(w)
        lw = LinearWeight("fp8", wq.data, wq.scale)
        xin = ops.quant_fp8(x)
        wbytes = n * k
    else:
        lw = LinearWeight("dense", w)
        xin = x
        wbytes = 2 * n * k
    if graph:
        lws = [lw] + [LinearWeight(lw.kind, lw.w.clone(), None if lw.scale_t is None else lw.scale_t.clone())
                      for _ in range(_copies(wbytes) - 1)]
        t = timed_graph([(lambda w_=w_: ops.linear(xin, w_)) for w_ in lws], reps)
    else:
        t = timed(lambda: ops.linear(xin, lw), reps)
    bw, fl, tag = peaks()
    bytes_ = wbytes + m * k * (1 if fp8 else 2) + 2 * m * n
    flops = 2.0 * m * n * k
    peak_fl = fl * (2 if fp8 else 1)
    roof = max(bytes_ / bw, flops / peak_fl)
    return {"op": "gemm", "m": m, "n": n, "k": k, "fp8": fp8, "us": t * 1e6, "GBps": bytes_ / t / 1e9,
            "TFLOPs": flops / t / 1e12, "roofline_us": roof * 1e6, "fraction": roof / t, "fraction_basis": tag}


def bench_gemm_w4(m, n, k, fmt, groups, reps, graph=False, a4=False, active=0, splits=0):
    """Dense (groups = 1) or grouped 4-bit-weight GEMM; grouped: m tokens spread evenly over the first `active` groups
    (all of them when 0).  a4: activations quantised to the weights' format and the block-scaled tensor-core kernel
    (the quantiser's launch is inside the timed call); otherwise the W4A16 kernel."""
    from ..ops.w4 import W4Weight, linear_w4, linear_w4a4
    dev = "cuda"
    g = max(1, groups)
    import numpy as np
    rng = np.random.default_rng(0)
    blk = 32 if fmt == "mxfp4" else 16
    packed = rng.integers(0, 256, (g, n, k // 2), dtype=np.uint8)
    scales = rng.integers(118, 126, (g, n, k // blk), dtype=np.uint8) if fmt == "mxfp4" else \
        rng.integers(0x30, 0x48, (g, n, k // blk), dtype=np.uint8)
    w = W4Weight.from_file_layout(fmt, packed, scales, k, None, dev)
    x = torch.randn(m, k, device=dev).bfloat16()
    off = None
    act = g if active <= 0 else min(active, g)
    mgt = m
    if g > 1:
        per = [m // act + (1 if i < m % act else 0) if i < act else 0 for i in range(g)]
        off = torch.tensor([0] + list(np.cumsum(per)), dtype=torch.int32, device=dev)
        mgt = max(per)
    if a4:
        w.native_tiles()
        call = lambda w_: linear_w4a4(x, w_, tok_off=off, max_group_tokens=mgt, splits=splits)
        wbytes = w.native.numel() * act // g
    else:
        call = lambda w_: linear_w4(x, w_, tok_off=off, max_group_tokens=mgt, splits=splits)
        wbytes = w.tiles.numel() * act // g
    if graph:
        ws = [w] + [W4Weight(w.fmt, w.groups, w.n, w.k, w.n_rows, w.k_pad, w.tiles if a4 else w.tiles.clone(), w.tensor_scale,
                             native=w.native.clone() if a4 else None)
                    for _ in range(_copies(wbytes) - 1)]
        t = timed_graph([(lambda w_=w_: call(w_)) for w_ in ws], reps)
    else:
        t = timed(lambda: call(w), reps)
    bw, fl, tag = peaks()
    bytes_ = wbytes + 2 * m * k + 2 * m * n
    flops = 2.0 * m * n * k
    roof = max(bytes_ / bw, flops / fl)
    return {"op": "gemm_w4a4" if a4 else "gemm_w4", "fmt": fmt, "m": m, "n": n, "k": k, "groups": g, "active_groups": act,
            "splits": splits, "us": t * 1e6, "GBps": bytes_ / t / 1e9,
            "TFLOPs": flops / t / 1e12, "roofline_us": roof * 1e6, "fraction": roof / t, "fraction_basis": tag}


def _kv(batch, ctx, hkv, hd, fp8, page=16):
    dev = "cuda"
    blocks = (ctx + page - 1) // page + 1
    pages = batch * blocks
    table = torch.arange(pages, device=dev, dtype=torch.int32).view(batch, blocks)
    if fp8:
        kv = KVLayer(torch.randint(0, 0x70, (pages, hkv, page, hd), device=dev, dtype=torch.uint8),
                     torch.randint(0, 0x70, (pages, hkv, page, hd), device=dev, dtype=torch.uint8),
                     torch.full((pages, hkv, page), 0.01, device=dev), torch.full((pages, hkv, page), 0.01, device=dev),
                     True, page)
    else:
        kv = KVLayer(torch.randn(pages, hkv, page, hd, device=dev).bfloat16(),
                     torch.randn(pages, hkv, page, hd, device=dev).bfloat16(), None, None, False, page)
    return kv, table


def bench_attention(batch, ctx, hq, hkv, hd, fp8, reps, graph=False):
    dev = "cuda"
    kv, table = _kv(batch, ctx, hkv, hd, fp8)
    q = torch.randn(batch, hq * hd, device=dev).bfloat16()
    seq = torch.arange(batch, device=dev, dtype=torch.int32)
    lens = torch.full((batch,), ctx, device=dev, dtype=torch.int32)
    bytes_ = 2 * batch * ctx * hkv * hd * (1 if fp8 else 2) + (2 * batch * ctx * hkv * 4 if fp8 else 0)
    call = lambda kv_: ops.paged_attention(q, kv_, table, seq, lens, hq, hkv, hd, max_kv=ctx, quant_out=fp8 and hd == 128)
    if graph:
        kvs = [kv] + [_kv(batch, ctx, hkv, hd, fp8)[0] for _ in range(_copies(bytes_) - 1)]
        t = timed_graph([(lambda kv_=kv_: call(kv_)) for kv_ in kvs], reps)
    else:
        t = timed(lambda: call(kv), reps)
    bw, _, tag = peaks()
    return {"op": "paged_attention", "batch": batch, "ctx": ctx, "hq": hq, "hkv": hkv, "hd": hd, "fp8": fp8,
            "us": t * 1e6, "GBps": bytes_ / t / 1e9, "roofline_us": bytes_ / bw * 1e6, "fraction": bytes_ / bw / t,
            "fraction_basis": tag}


def bench_prefill(seqs, length, hq, hkv, reps):
    from ..engine.batch import make_prefill_batch
    from ..ops import prefill
    dev = "cuda"
    hd = 128
    t_tok = seqs * length
    qkv = torch.randn(t_tok, (hq + 2 * hkv) * hd, device=dev).bfloat16()
    table = torch.zeros((seqs, 1), dtype=torch.int32, device=dev)
    b = make_prefill_batch([[0] * length] * seqs, table, dev)
    t = timed(lambda: prefill.prefill_attention(qkv, b, hq, hkv, hd), reps)
    _, fl, tag = peaks()
    flops = 4.0 * seqs * hq * hd * length * (length + 1) / 2
    return {"op": "prefill_attention", "seqs": seqs, "len": length, "hq": hq, "hkv": hkv, "us": t * 1e6,
            "TFLOPs": flops / t / 1e12, "fraction": flops / fl / t, "fraction_basis": tag}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["gemm", "gemm-w4", "attention", "prefill", "decode-gemms"])
    ap.add_argument("--fmt", default="nvfp4", choices=["nvfp4", "mxfp4"])
    ap.add_argument("--groups", type=int, default=1)
    ap.add_argument("--active", type=int, default=0, help="gemm-w4, grouped: groups that receive tokens (0 = all)")
    ap.add_argument("--splits", type=int, default=0, help="gemm-w4: K splits (0 = the wrapper's choice)")
    ap.add_argument("--a4", action="store_true", help="gemm-w4: 4-bit activations on the block-scaled tensor-core kernel")
    ap.add_argument("--m", type=int, default=32)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--fp8", action="store_true")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--hd", type=int, default=128)
    ap.add_argument("--seqs", type=int, default=4)
    ap.add_argument("--len", type=int, default=2048)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--graph", action="store_true",
                    help="time back-to-back launches over distinct buffers inside one CUDA graph (steady state)")
    a = ap.parse_args()
    if a.op == "gemm":
        print(json.dumps(bench_gemm(a.m, a.n, a.k, a.fp8, a.reps, a.graph)))
    elif a.op == "gemm-w4":
        print(json.dumps(bench_gemm_w4(a.m, a.n, a.k, a.fmt, a.groups, a.reps, a.graph, a.a4, a.active, a.splits)))
    elif a.op == "attention":
        print(json.dumps(bench_attention(a.batch, a.ctx, a.hq, a.hkv, a.hd, a.fp8, a.reps, a.graph)))
    elif a.op == "prefill":
        print(json.dumps(bench_prefill(a.seqs, a.len, a.hq, a.hkv, a.reps)))
    else:
        for (n, k) in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (128256, 4096)):
            print(json.dumps(bench_gemm(a.m, n, k, True, a.reps, a.graph)))


if __name__ == "__main__":
    main()

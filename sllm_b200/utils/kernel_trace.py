"""Per-tile / per-chunk cycle timelines of the pipelined tensor-core kernels: the tracing tool of the kernel library.

The kernels carry `clock64` stamps of CTA (0,0,0) that compile in only under `-DSLLM_TRACE`.  This tool builds a
trace-instrumented copy of the kernel library into a temporary directory, runs one cold launch and prints the
stamps relative to the first one, one line per 128-key tile (decode attention) or per 128-element K chunk
(W4 GEMM).  The product library is never built with the stamps.

    python -m sllm_b200.utils.kernel_trace --op attention --batch 32 --ctx 2048
    python -m sllm_b200.utils.kernel_trace --op gemm-w4 --fmt nvfp4 --n 28672 --k 8192
    python -m sllm_b200.utils.kernel_trace --op fused-decode --batch 32          # per-phase stamps of the persistent kernel

With ``--json`` the result is one JSON object (schema ``sllm-kernel-trace-v1``): ``op``, ``shape``, ``cold_us``,
``columns`` (stamp names) and ``rows`` (one list per tile / chunk / phase; clock cycles, or nanoseconds for
fused-decode, relative to the earliest stamp; null where a stamp was not taken).

Columns, decode attention (softmax thread 0 unless noted): top = loop top, s_full = S ready, ld = S read from
TMEM, sync = maxima exchanged, arrive = P written and announced, fold = previous P.V folded; S_go / S_done and
PV_go / PV_done = the issuer threads before / after their four MMAs.
Columns, W4 GEMM: p_empty / p_issued = producer passed the stage-free wait / issued the copies; m_convdone /
m_issued = issuer saw the converted tile / issued its MMAs; c_full = converter saw the stage's data, c_aempty =
its output buffer is free, c_conv = conversion done, c_arrived = fence + arrivals done.
"""
from __future__ import annotations

import argparse
import ctypes as C
import glob
import os
import pathlib
import subprocess
import tempfile


def _build_traced() -> str:
    here = pathlib.Path(__file__).resolve().parent.parent / "csrc"
    out = tempfile.mkdtemp(prefix="sllm_trace_")
    objs = []
    for src in sorted(glob.glob(str(here / "*.cu"))):
        obj = os.path.join(out, os.path.basename(src) + ".o")
        subprocess.check_call(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17",
                               "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-DSLLM_TRACE", f"-I{here}", "-c", src,
                               "-o", obj], stderr=subprocess.DEVNULL)
        objs.append(obj)
    lib = os.path.join(out, "libsllm_b200_traced.so")
    subprocess.check_call(["nvcc", "-shared", "-o", lib, *objs, "-lcudart", "-lcuda"])
    return lib


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["attention", "gemm-w4", "fused-decode"])
    ap.add_argument("--json", action="store_true", help="print one sllm-kernel-trace-v1 JSON object instead of text")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--fmt", default="nvfp4", choices=["nvfp4", "mxfp4"])
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=28672)
    ap.add_argument("--k", type=int, default=8192)
    a = ap.parse_args(argv)
    import json
    import torch
    from ..ops import _lib
    if a.op == "fused-decode":
        return _fused_decode(a)
    _lib._KERNEL_PATH = pathlib.Path(_build_traced())
    lib = _lib.kernels()
    dev = "cuda"

    def cold(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        junk = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        junk.zero_()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1000

    if a.op == "attention":
        from .. import ops
        from .kernel_bench import _kv
        hq, hkv, hd = 32, 8, 128
        kv, table = _kv(a.batch, a.ctx, hkv, hd, True)
        q = torch.randn(a.batch, hq * hd, device=dev).bfloat16()
        seq = torch.arange(a.batch, device=dev, dtype=torch.int32)
        lens = torch.full((a.batch,), a.ctx, device=dev, dtype=torch.int32)
        us = cold(lambda: ops.paged_attention(q, kv, table, seq, lens, hq, hkv, hd, max_kv=a.ctx, quant_out=True))
        tr = (C.c_longlong * 256)()
        lib.sllm_decode_attention_read_trace(tr)
        names = ["top", "s_full", "ld", "sync", "arrive", "fold", "S_go", "PV_go", "S_done", "PV_done"]
        shape = {"batch": a.batch, "ctx": a.ctx}
        rows, per = min(24, (a.ctx + 127) // 128), 10
    else:
        import numpy as np
        from ..ops.w4 import W4Weight, linear_w4
        rng = np.random.default_rng(0)
        blk = 16 if a.fmt == "nvfp4" else 32
        lo, hi = (0x30, 0x48) if a.fmt == "nvfp4" else (118, 128)
        w = W4Weight.from_file_layout(a.fmt, rng.integers(0, 256, (1, a.n, a.k // 2), dtype=np.uint8),
                                      rng.integers(lo, hi, (1, a.n, a.k // blk), dtype=np.uint8), a.k, None, dev)
        x = torch.randn(a.m, a.k, device=dev).bfloat16()
        us = cold(lambda: linear_w4(x, w))
        tr = (C.c_longlong * 1024)()
        lib.sllm_gemm_w4_read_trace(tr)
        names = ["p_empty", "p_issued", "m_convdone", "m_issued", "c_full", "c_aempty", "c_conv", "c_arrived"]
        shape = {"fmt": a.fmt, "m": a.m, "n": a.n, "k": a.k}
        rows, per = min(24, a.k // 128), 10
    t0 = min(v for v in tr if v > 0)
    table = []
    for j in range(rows):
        vals = [tr[j * per + i] for i in range(len(names))]
        if not any(v > 0 for v in vals):
            break
        table.append([v - t0 if v > 0 else None for v in vals])
    _emit(a, {"schema": "sllm-kernel-trace-v1", "op": a.op, "shape": shape, "cold_us": round(us, 2), "columns": names,
              "rows": table})
    return 0


def _emit(a, doc: dict) -> None:
    import json
    if a.json:
        print(json.dumps(doc))
        return
    print(f"{doc['op']} {doc['shape']}: {doc['cold_us']} us cold")
    for j, row in enumerate(doc["rows"]):
        print(j, " ".join(f"{n}={'-' if v is None else v}" for n, v in zip(doc["columns"], row)))


def _fused_decode(a) -> int:
    """Per-phase stamps (nanoseconds, earliest and latest CTA) of one launch of the persistent fused decode kernel at
    Llama-3-8B layer shapes: o-projection, gate/up, down, q/k/v.  Uses the library's own trace switch; no rebuild."""
    import torch
    from ..ops import fused_decode as fd
    from ..ops.core import KVLayer
    dev = torch.device("cuda")
    rows = min(a.batch, 32)
    bn = 16 if rows <= 16 else 32
    d, qs, ffn, nq = 4096, 4096, 14336, 6144

    def w(n, k):
        return (torch.empty((n, k), dtype=torch.uint8, device=dev).random_(0, 120), torch.rand((k // 128, n), device=dev) * 0.01 + 0.001)

    def x(k):
        return (torch.empty((rows, k), dtype=torch.uint8, device=dev).random_(0, 120), torch.rand((k // 128, bn), device=dev) * 0.01 + 0.001)

    z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=dev)
    (wo, so), (wgu, sgu), (wd, sd), (wq, sq) = w(d, qs), w(2 * ffn, d), w(d, ffn), w(nq, d)
    aq, a_s = x(qs)
    h = (torch.randn(rows, d, device=dev) * 0.5).bfloat16()
    hq, hs, ssq = z((rows, d), torch.uint8), z((d // 128, bn), torch.float32), torch.ones((d // 128, bn), device=dev)
    actq, acts, qout = z((rows, ffn), torch.uint8), z((ffn // 128, bn), torch.float32), z((rows, 4096), torch.bfloat16)
    pages = rows * 8
    kv = KVLayer(z((pages, 8, 16, 128), torch.uint8), z((pages, 8, 16, 128), torch.uint8), z((pages, 8, 16), torch.float32),
                 z((pages, 8, 16), torch.float32), True, 16)
    pos = torch.full((rows,), 37, dtype=torch.int32, device=dev)
    si = torch.arange(rows, dtype=torch.int32, device=dev)
    bt = torch.arange(rows * 8, dtype=torch.int32, device=dev).view(rows, 8)
    phases = [
        fd.phase(fd.RESID_QUANT, wo, so, aq, a_s, n=d, k=qs, y=h, ldy=d, residual=h, q_out=hq, s_out=hs, ssq_out=ssq, ld_s_out=bn),
        fd.phase(fd.SILU_QUANT, wgu, sgu, hq, hs, n=ffn, k=d, dual_off=ffn, ssq_in=ssq, norm_dim=d, q_out=actq, s_out=acts, ld_s_out=bn),
        fd.phase(fd.RESID_QUANT, wd, sd, actq, acts, n=d, k=ffn, y=h, ldy=d, residual=h, q_out=hq, s_out=hs, ssq_out=ssq, ld_s_out=bn),
        fd.phase(fd.ROPE_KV, wq, sq, hq, hs, n=nq, k=d, ssq_in=ssq, norm_dim=d, y=qout, ldy=4096, ld_s_out=bn)]
    rope = fd.rope_desc(pos, si, bt, kv, 32, 8, 128, 500000.0)
    for _ in range(3):
        fd.launch(phases, rows, dev, rope, impl="persistent")
    torch.cuda.synchronize()
    ctas = torch.cuda.get_device_properties(dev).multi_processor_count
    tr = torch.zeros((ctas, 4, 8), dtype=torch.int64, device=dev)
    fd.set_trace(tr)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fd.launch(phases, rows, dev, rope, impl="persistent")
    e1.record()
    torch.cuda.synchronize()
    fd.set_trace(None)
    t = tr.cpu()
    t0 = int(t[:, 0, 0][t[:, 0, 0] > 0].min())
    names = ["setup", "input_visible", "first_accumulator", "promoted", "tile_complete", "outputs_written", "barrier_arrival"]
    cols, table = [], []
    for n in names:
        cols += [n + ".first", n + ".last"]
    for pi in range(4):
        row = []
        for s in range(7):
            v = t[:, pi, s][t[:, pi, s] > 0]
            row += [None, None] if v.numel() == 0 else [int(v.min()) - t0, int(v.max()) - t0]
        table.append(row)
    _emit(a, {"schema": "sllm-kernel-trace-v1", "op": "fused-decode", "shape": {"rows": rows, "model": "llama3-8b layer"},
              "cold_us": round(e0.elapsed_time(e1) * 1000, 2), "columns": cols, "rows": table})
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

"""Per-tile / per-chunk cycle timelines of the two pipelined tensor-core kernels (development aid).

The kernels carry `clock64` stamps of CTA (0,0,0) that compile in only under `-DSLLM_TRACE`.  This tool builds a
trace-instrumented copy of the kernel library into a temporary directory, runs one cold launch and prints the
stamps relative to the first one, one line per 128-key tile (decode attention) or per 128-element K chunk
(W4 GEMM).  The product library is never built with the stamps.

    python -m sllm_b200.utils.kernel_trace --op attention --batch 32 --ctx 2048
    python -m sllm_b200.utils.kernel_trace --op gemm-w4 --fmt nvfp4 --n 28672 --k 8192

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
    ap.add_argument("--op", required=True, choices=["attention", "gemm-w4"])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--fmt", default="nvfp4", choices=["nvfp4", "mxfp4"])
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=28672)
    ap.add_argument("--k", type=int, default=8192)
    a = ap.parse_args(argv)
    import torch
    from ..ops import _lib
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
        print(f"decode attention batch={a.batch} ctx={a.ctx}: {us:.1f} us cold")
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
        print(f"gemm_w4 {a.fmt} m={a.m} n={a.n} k={a.k}: {us:.1f} us cold")
        rows, per = min(24, a.k // 128), 10
    t0 = min(v for v in tr if v > 0)
    for j in range(rows):
        vals = [tr[j * per + i] for i in range(len(names))]
        if not any(v > 0 for v in vals):
            break
        print(j, " ".join(f"{n}={v - t0 if v > 0 else '-'}" for n, v in zip(names, vals)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

"""Device-timed comparison of the fused compute+collective kernels with their NCCL counterparts.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m sllm_b200.utils.comm_bench [--rows 32] [--d 4096] [--ffn 14336] [--iters 50]

Three pairs, Llama-3-8B decode shapes by default, bf16, one line of JSON per pair from rank 0:
  row_linear      row-parallel GEMM [rows, ffn / N] x [d, ffn / N]^T + all-reduce (fused: tiles pushed into every
                  rank's receive buffer from the GEMM epilogue) vs GEMM + ncclAllReduce
  gather_linear   all-gather of K shards [rows, d / N] + column-parallel GEMM [2 ffn / N, d] (fused: the GEMM's TMA
                  producer pulls the peers' shards) vs ncclAllGather + GEMM
  ep_combine      expert-parallel combine of rows x top-4 expert outputs (fused: weighted sum + cross-rank sum in one
                  kernel over peer memory) vs local combine + ncclAllReduce
  ep_experts      the whole MoE block after routing at the 120B-class expert shape (permute, gather, grouped MXFP4
                  gate_up, SiLU*up, grouped down projection, combine): token-owner path (rows leave the down-projection
                  epilogue for their owner's slots, owners sum and gather) vs the all-reduce form (every rank pushes a
                  full partial to every peer) vs local combine + ncclAllReduce
Times are CUDA events around one replay of a CUDA graph that holds `iters` back-to-back calls (`--eager` times eager
calls instead), after warm-up, max over ranks.  The roofline of a pair is the
slower of (weight bytes / measured copy bandwidth) and (bytes that must cross NVLink per GPU / 770 GB/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

HBM_GBS_FALLBACK = 6650.0
NVLINK_GBS = 770.0


def _hbm_gbs():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "of measured"
    except Exception:
        return HBM_GBS_FALLBACK, "of fallback"


_EAGER = [False]


def _time(fn, iters: int, warmup: int = 5) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if _EAGER[0]:
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
    else:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(iters):
                    fn()
            g.replay()                      # first replay: uploads the graph
            side.synchronize()
            dist.barrier()
            e0.record(side)
            g.replay()
            e1.record(side)
            side.synchronize()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1000.0 / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=32)
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of a CUDA graph replay")
    ap.add_argument("--moe-rows", type=int, default=64)
    a = ap.parse_args(argv)
    _EAGER[0] = a.eager
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from .. import ops
    from ..ops.core import LinearWeight
    from ..parallel.ep import FusedEP, NcclEP
    from ..parallel.gather import GatherGemm, NcclGatherGemm
    from ..parallel.tp import make_tp
    hbm, basis = _hbm_gbs()
    m, d, f = a.rows, a.d, a.ffn
    gen = torch.Generator(device=dev).manual_seed(rank)

    def rnd(*shape, s=0.05):
        return (torch.randn(*shape, device=dev, generator=gen) * s).bfloat16()

    out = []
    # ---- row-parallel GEMM + all-reduce
    fs = f // world // 64 * 64
    w_row = LinearWeight("dense", rnd(d, fs))
    x_row, res = rnd(m, fs, s=1.0), rnd(m, d, s=1.0)
    fused_tp = make_tp(world, rank, dev, impl="fused", max_tokens=max(m, 128), d_model=d)
    nccl_tp = make_tp(world, rank, dev, impl="nccl")
    t_f = _time(lambda: fused_tp.row_linear(x_row, w_row, res), a.iters)
    t_n = _time(lambda: nccl_tp.row_linear(x_row, w_row, res), a.iters)
    link_bytes = m * d * 2 * (world - 1)                   # every rank's partial goes to every other rank
    roof = max(d * fs * 2 / hbm / 1e3, link_bytes / NVLINK_GBS / 1e3)
    out.append({"op": "row_linear", "fused_us": t_f, "nccl_us": t_n, "roofline_us": roof, "weight_mb": d * fs * 2 / 1e6,
                "nvlink_bytes_per_gpu": link_bytes})
    # ---- all-gather + column-parallel GEMM
    n_loc = 2 * f // world // 128 * 128
    w_col = LinearWeight("dense", rnd(n_loc, d))
    shard = rnd(m, d // world, s=1.0)
    gg, ng = GatherGemm(world, rank, dev, max_rows=max(m, 16), k=d), NcclGatherGemm(world, rank, dev)
    t_f = _time(lambda: gg.linear(shard, w_col), a.iters)
    t_n = _time(lambda: ng.linear(shard, w_col), a.iters)
    link_bytes = m * (d // world) * 2 * (world - 1)
    roof = max(n_loc * d * 2 / hbm / 1e3, link_bytes / NVLINK_GBS / 1e3)
    out.append({"op": "gather_linear", "fused_us": t_f, "nccl_us": t_n, "roofline_us": roof,
                "weight_mb": n_loc * d * 2 / 1e6, "nvlink_bytes_per_gpu": link_bytes})
    # ---- expert-parallel combine
    top_k = 4
    fe, ne = FusedEP(world, rank, dev, max(m, 128), d), NcclEP(world, rank, dev)
    pairs = m * top_k
    idx = torch.arange(pairs, device=dev, dtype=torch.int32).view(m, top_k)
    mine = (idx % world) == rank                            # the pairs whose expert lives on this rank
    rows_local = int(mine.sum().item())
    yp = rnd(max(rows_local, 1), d, s=1.0)
    dst = torch.full((m, top_k), -1, dtype=torch.int32, device=dev)
    dst[mine] = torch.arange(rows_local, device=dev, dtype=torch.int32)
    t_f = _time(lambda: fe.combine(yp, dst, res), a.iters)
    t_n = _time(lambda: ne.combine(yp, dst, res), a.iters)
    link_bytes = m * d * 2 * (world - 1)
    out.append({"op": "ep_combine", "fused_us": t_f, "nccl_us": t_n, "roofline_us": link_bytes / NVLINK_GBS / 1e3,
                "nvlink_bytes_per_gpu": link_bytes})
    # ---- the MoE block after routing, 120B-class expert shape (d 2880, expert ffn 2880, 128 experts, top-4, MXFP4)
    from ..ops import moe as M
    from ..ops.w4 import W4Weight
    md, mf, n_exp, mk, rows = 2880, 2880, 128, 4, a.moe_rows
    per = n_exp // world
    e_lo, e_hi = rank * per, (rank + 1) * per
    g2 = torch.Generator(device=dev).manual_seed(100 + rank)
    gate_up = W4Weight.quantize_device("mxfp4", (torch.randn(per, 2 * mf, md, device=dev, generator=g2) * 0.02).bfloat16())
    down = W4Weight.quantize_device("mxfp4", (torch.randn(per, md, mf, device=dev, generator=g2) * 0.02).bfloat16())
    gx = torch.Generator(device=dev).manual_seed(7)          # the same tokens and routing on every rank
    xm = (torch.randn(rows, md, device=dev, generator=gx)).bfloat16()
    resm = (torch.randn(rows, md, device=dev, generator=gx)).bfloat16()
    idx_m, rw_m = M.route((torch.randn(rows, n_exp, device=dev, generator=gx)).bfloat16(), mk)
    fo = FusedEP(world, rank, dev, max(rows, 128), md)
    t_o = _time(lambda: fo.experts_combine(xm, idx_m, rw_m, gate_up, down, "silu", e_lo, e_hi, resm), a.iters)
    fo.owner_path = False
    t_a = _time(lambda: fo.experts_combine(xm, idx_m, rw_m, gate_up, down, "silu", e_lo, e_hi, resm), a.iters)
    t_n = _time(lambda: ne.experts_combine(xm, idx_m, rw_m, gate_up, down, "silu", e_lo, e_hi, resm), a.iters)
    mine_rows = int(((idx_m >= e_lo) & (idx_m < e_hi)).sum().item())
    tpr = (rows + world - 1) // world
    owner_bytes = (mine_rows + tpr * (world - 1)) * md * 2       # routed rows to their owners (upper bound: all remote) + own tokens to every peer
    w_bytes = (gate_up.nbytes() + down.nbytes())
    out.append({"op": "ep_experts", "fused_us": t_o, "allreduce_form_us": t_a, "nccl_us": t_n,
                "roofline_us": max(w_bytes / hbm / 1e3, owner_bytes / NVLINK_GBS / 1e3), "weight_mb": w_bytes / 1e6,
                "nvlink_bytes_per_gpu": owner_bytes, "nvlink_bytes_per_gpu_allreduce_form": rows * md * 2 * (world - 1),
                "rows": rows, "top_k": mk, "experts_per_rank": per})
    status = ops.device_status(dev)
    torch.cuda.synchronize()
    fo.close()
    gg.close()
    fe.close()
    fused_tp.close()
    if rank == 0:
        for o in out:
            o.setdefault("rows", m)
            o.setdefault("d", d)
            o.update({"world": world, "timed": "eager" if a.eager else "graph replay",
                      "speedup_vs_nccl": round(o["nccl_us"] / o["fused_us"], 3),
                      "fraction_of_roofline": round(o["roofline_us"] / o["fused_us"], 3), "fraction_basis": basis,
                      "device_status": status})
            if "allreduce_form_us" in o:
                o["allreduce_form_us"] = round(o["allreduce_form_us"], 2)
            o["fused_us"], o["nccl_us"], o["roofline_us"] = (round(o[k], 2) for k in ("fused_us", "nccl_us", "roofline_us"))
            print(json.dumps(o), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

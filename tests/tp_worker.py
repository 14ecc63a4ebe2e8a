"""Per-rank body of the tensor-parallel GPU tests (launched by test_tp_gpu.py through torchrun)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from sllm_b200 import ops  # noqa: E402
from sllm_b200.engine.engine import build_engine  # noqa: E402
from sllm_b200.models.config import ModelConfig  # noqa: E402
from sllm_b200.ops.core import LinearWeight  # noqa: E402
from sllm_b200.parallel.tp import make_tp  # noqa: E402


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import datetime
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))

    def mark(msg):
        if os.environ.get("SLLM_TEST_VERBOSE"):
            print(f"[rank {rank}] {msg}", flush=True)

    d_model = 1024
    fused = make_tp(world, rank, dev, impl="fused", max_tokens=256, d_model=d_model)
    nccl = make_tp(world, rank, dev, impl="nccl")
    torch.manual_seed(0)  # same full tensors on every rank
    for kind in ("dense", "fp8"):
        for m in (1, 7, 32, 64, 100, 200):
            k_full = 2048
            x = torch.randn(m, k_full, device=dev).bfloat16()
            w = (torch.randn(d_model, k_full, device=dev) * 0.03).bfloat16()
            r = torch.randn(m, d_model, device=dev).bfloat16()
            ks = k_full // world
            xs = x[:, rank * ks:(rank + 1) * ks].contiguous()
            ws = w[:, rank * ks:(rank + 1) * ks].contiguous()
            lw = LinearWeight.from_dense(ws.cpu(), kind).to(dev) if kind == "fp8" else LinearWeight("dense", ws)
            want = x.float() @ w.float().t() + r.float()
            for rep in range(3):  # repeated calls with different data exercise the double-buffered regions
                junk = fused.row_linear((xs.float() * (rep + 2)).bfloat16() if kind == "dense" else xs, lw, r)
            y_f = fused.row_linear(xs, lw, r)
            y_n = nccl.row_linear(xs, lw, r)
            tol = 6e-2 if kind == "fp8" else 1.2e-2
            assert rel(y_f, want) < tol, (kind, m, rel(y_f, want))
            assert rel(y_f, y_n) < 1.5e-2, (kind, m, rel(y_f, y_n))
            # every rank must hold bit-identical results
            parts = [torch.empty_like(y_f) for _ in range(world)]
            dist.all_gather(parts, y_f)
            for p in parts:
                assert torch.equal(p, parts[0]), (kind, m, "ranks disagree")
    # 4-bit weights: W4A16 GEMM + the fused peer-memory row reduction
    from sllm_b200.ops.w4 import W4Weight
    for m in (3, 40):
        x = torch.randn(m, 1024, device=dev).bfloat16()
        w = (torch.randn(d_model, 1024, device=dev) * 0.03)
        r = torch.randn(m, d_model, device=dev).bfloat16()
        dist.broadcast(x, 0); dist.broadcast(w, 0); dist.broadcast(r, 0)
        ks = 1024 // world
        lw = LinearWeight("w4", None, None, W4Weight.quantize_device("nvfp4", w[:, rank * ks:(rank + 1) * ks].contiguous()))
        full = W4Weight.quantize_device("nvfp4", w)   # per-shard tensor scales differ slightly: compare loosely
        want = x.float() @ full.dequantized(0).to(dev).t() + r.float()
        xs = x[:, rank * ks:(rank + 1) * ks].contiguous()
        y_f = fused.row_linear(xs, lw, r)
        y_n = nccl.row_linear(xs, lw, r)
        assert rel(y_f, want) < 0.15 and rel(y_f, y_n) < 1.5e-2, (m, rel(y_f, want), rel(y_f, y_n))
    mark("row_linear ok")
    # vocabulary-parallel argmax
    logits = torch.randn(5, 4096, device=dev).bfloat16()
    dist.broadcast(logits, 0)
    vs = 4096 // world
    shard = logits[:, rank * vs:(rank + 1) * vs].contiguous()
    got = fused.argmax(shard, rank * vs)
    assert torch.equal(got.cpu(), logits.float().argmax(-1).int().cpu()), (got, logits.float().argmax(-1))
    assert ops.device_status(dev) == 0

    # end to end: TP engine reproduces the single-GPU greedy tokens
    cfg = ModelConfig(name="tp-test", n_layers=2, d_model=d_model, n_heads=8, n_kv_heads=4, head_dim=128, ffn=2048,
                      vocab=4096, weight_format="fp8", kv_format="fp8", max_context=256)
    g = torch.Generator().manual_seed(5)
    prompts = torch.randint(0, cfg.vocab, (3, 40), generator=g).tolist()
    mark("argmax ok")
    ref_eng = build_engine(cfg, dev, seed=1, max_batch=4)
    ref_seqs = [ref_eng.new_sequence(p) for p in prompts]
    want_logits = ref_eng.prefill(ref_seqs, sample=False).float()
    first = want_logits.argmax(-1).tolist()
    for s, t in zip(ref_seqs, first):
        s.tokens.append(t)
    want_decode = ref_eng.decode(ref_seqs, sample=False).float().clone()      # one decode step (the fused decode path)
    for tp in (fused, nccl):
        mark(f"building {tp.impl} engine")
        eng = build_engine(cfg, dev, seed=1, max_batch=4, tp=tp)
        seqs = [eng.new_sequence(p) for p in prompts]
        got_logits = eng.prefill(seqs, sample=False).float()
        assert got_logits.shape == want_logits.shape
        assert rel(got_logits, want_logits) < 0.12, (tp.impl, rel(got_logits, want_logits))  # fp8 model, bf16 partial sums
        # decode step of the same sequences: with the fused communicator this is the fused decode chain, whose
        # row-parallel phases sum their tiles across ranks inside the kernel
        for s, t in zip(seqs, first):
            s.tokens.append(t)
        got_decode = eng.decode(seqs, sample=False).float()
        assert rel(got_decode, want_decode) < 0.12, (tp.impl, "decode", rel(got_decode, want_decode))
        if tp.impl == "fused":
            assert bool(eng.model._fused), "the tensor-parallel decode step did not take the fused chain"
        for s in seqs:
            eng.free_sequence(s)
        mark(f"{tp.impl} prefill logits ok")
        # greedy decoding (different records every step): every rank must produce the same tokens
        got_tokens = eng.generate(prompts, 12, on_token=lambda i, t: mark(f"tok {i} {t}"))
        mark(f"{tp.impl} generate done")
        obj = [None] * world
        dist.all_gather_object(obj, got_tokens)
        assert all(o == obj[0] for o in obj), ("ranks produced different tokens", tp.impl, obj)
    assert ops.device_status(dev) == 0
    del eng, ref_eng
    torch.cuda.synchronize()
    # all-gather fused into a column-parallel GEMM: K shards pulled from the peers by the GEMM's own TMA producer
    from sllm_b200.parallel.gather import GatherGemm, NcclGatherGemm
    k, n_local = 512 * world, 384
    gg = GatherGemm(world, rank, dev, max_rows=200, k=k)
    ng = NcclGatherGemm(world, rank, dev)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    w_local = LinearWeight("dense", (torch.randn(n_local, k, device=dev, generator=gen) * 0.05).bfloat16())
    for m in (1, 5, 33, 128, 200):
        for rep in range(3):                      # both buffer parities
            x = (torch.randn(m, k, device=dev) * (rep + 1)).bfloat16()
            dist.broadcast(x, 0)
            res = torch.randn(m, n_local, device=dev).bfloat16()
            shard = x[:, rank * (k // world):(rank + 1) * (k // world)]
            want = x.float() @ w_local.w.float().t() + res.float()
            got_f = gg.linear(shard, w_local, res)
            got_n = ng.linear(shard, w_local, res)
            assert rel(got_f, want) < 1e-2, ("gather fused", m, rep, rel(got_f, want))
            assert rel(got_n, want) < 1e-2, ("gather nccl", m, rep, rel(got_n, want))
    assert ops.device_status(dev) == 0
    mark("gather gemm ok")
    torch.cuda.synchronize()
    gg.close()
    fused.close()
    dist.barrier()
    if rank == 0:
        print("TP_WORKER_OK", flush=True)
    mark("destroying process group")
    dist.destroy_process_group()
    mark("exiting")
    sys.stdout.flush()
    os._exit(0)  # skip interpreter teardown of CUDA graphs that captured library collectives


if __name__ == "__main__":
    main()

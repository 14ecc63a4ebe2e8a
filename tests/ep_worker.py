"""Per-rank body of the expert-parallel GPU test (launched by test_tp_gpu.py through torchrun)."""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from sllm_b200 import ops  # noqa: E402
from sllm_b200.cache.paged import PagedKVCache  # noqa: E402
from sllm_b200.engine.engine import Engine  # noqa: E402
from sllm_b200.models import moe as MOE  # noqa: E402
from sllm_b200.ops import moe as M  # noqa: E402
from sllm_b200.parallel.ep import FusedEP, NcclEP  # noqa: E402
from sllm_b200.parallel.tp import make_tp  # noqa: E402


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    cfg = MOE.tiny_moe()
    cfg.n_experts, cfg.top_k = 8, 2
    if world > cfg.n_kv_heads:            # the attention of the end-to-end part is sharded by head over all ranks
        cfg.n_heads, cfg.n_kv_heads = 2 * world, world
    d = cfg.d_model
    fused = FusedEP(world, rank, dev, max_tokens=64, d_model=d)
    nccl = NcclEP(world, rank, dev)
    full = MOE.init_random_moe_weights(cfg, dev, seed=2).layers[0]
    mine = MOE.init_random_moe_weights(cfg, dev, seed=2, ep_size=world, ep_rank=rank).layers[0]
    e_lo, e_hi = nccl.expert_range(cfg.n_experts)
    torch.manual_seed(1)
    for t in (1, 5, 33, 64):
        for rep in range(3):                       # repeated calls exercise both parities of the receive slots
            x = torch.randn(t, d, device=dev).bfloat16() * (rep + 1)
            dist.broadcast(x, 0)
            res = torch.randn(t, d, device=dev).bfloat16()
            dist.broadcast(res, 0)
            idx, rw = M.route(ops.linear(x, full.router), cfg.top_k)
            yp, dst = M.experts_forward(x, idx, rw, full.gate_up, full.down, cfg.act, 0, cfg.n_experts)
            want = M.combine(yp, dst, res)
            yp_r, dst_r = M.experts_forward(x, idx, rw, mine.gate_up, mine.down, cfg.act, e_lo, e_hi)
            got_f = fused.combine(yp_r, dst_r, res)
            got_n = nccl.combine(yp_r, dst_r, res)
            assert rel(got_f, want) < 1.5e-2, (t, rep, rel(got_f, want))
            assert rel(got_n, want) < 1.5e-2, (t, rep, rel(got_n, want))
            parts = [torch.empty_like(got_f) for _ in range(world)]
            dist.all_gather(parts, got_f)
            for p in parts:
                assert torch.equal(p, parts[0]), "ranks disagree"
            # token-owner path: rows leave the down-projection epilogue for their owner, owners sum and gather
            got_o = fused.experts_combine(x, idx, rw, mine.gate_up, mine.down, cfg.act, e_lo, e_hi, res)
            assert rel(got_o, want) < 1.5e-2, ("owner", t, rep, rel(got_o, want))
            dist.all_gather(parts, got_o)
            for p in parts:
                assert torch.equal(p, parts[0]), "ranks disagree (owner path)"
    assert ops.device_status(dev) == 0
    # end to end: EP + TP MoE engine reproduces the single-GPU greedy tokens on every rank
    g = torch.Generator().manual_seed(5)
    prompts = torch.randint(0, cfg.vocab, (3, 24), generator=g).tolist()

    def engine(tp=None, ep=None):
        w = MOE.init_random_moe_weights(cfg, dev, seed=3, tp_size=tp.size if tp else 1, tp_rank=tp.rank if tp else 0,
                                        ep_size=ep.size if ep else 1, ep_rank=ep.rank if ep else 0)
        model = MOE.MoeModel(cfg, w, tp=tp, ep=ep)
        cache = PagedKVCache(cfg, 64, dev, kv_heads=model.local_kv_heads)
        return Engine(cfg, model, cache, dev, max_batch=4, tp=tp)

    ref_eng = engine()
    want_logits = ref_eng.prefill([ref_eng.new_sequence(p) for p in prompts], sample=False).float()
    tp = make_tp(world, rank, dev, impl="fused", max_tokens=256, d_model=d)
    eng = engine(tp, fused)
    got_logits = eng.prefill([eng.new_sequence(p) for p in prompts], sample=False).float()
    assert rel(got_logits, want_logits) < 0.08, rel(got_logits, want_logits)
    toks = eng.generate(prompts, 8)
    obj = [None] * world
    dist.all_gather_object(obj, toks)
    assert all(o == obj[0] for o in obj), "ranks produced different tokens"
    assert ops.device_status(dev) == 0
    del eng, ref_eng
    torch.cuda.synchronize()
    fused.close()
    tp.close()
    dist.barrier()
    if rank == 0:
        print("EP_WORKER_OK", flush=True)
    dist.destroy_process_group()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()

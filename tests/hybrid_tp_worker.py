"""Tensor-parallel gated-delta-net hybrid on CPU (gloo): two ranks, heads and MLP channels sharded, must reproduce
the single-rank logits and greedy tokens (launched by test_model_families.py through torchrun)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from sllm_b200.engine.engine import build_engine  # noqa: E402
from sllm_b200.models.qwen35 import tiny_qwen35  # noqa: E402
from sllm_b200.parallel.tp import NcclTP  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    cfg = tiny_qwen35()
    cfg.weight_format, cfg.kv_format = "fp32", "fp32"
    cfg.n_kv_heads, cfg.gdn_qk_heads, cfg.gdn_heads = 2, 2, 4     # one KV head, one q/k head, two value heads per rank
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (9, 17, 5)]
    ref = build_engine(cfg, "cpu", seed=2, max_batch=4, use_cuda_graphs=False)
    want_logits = ref.prefill([ref.new_sequence(p) for p in prompts], sample=False).clone()
    want_tokens = build_engine(cfg, "cpu", seed=2, max_batch=4, use_cuda_graphs=False).generate(prompts, 8)
    tp = NcclTP(world, rank, torch.device("cpu"))
    eng = build_engine(cfg, "cpu", seed=2, max_batch=4, use_cuda_graphs=False, tp=tp)
    # each rank holds its share of the state and of the weights
    assert eng.cache.rec_state.shape[2] == cfg.gdn_heads // world
    assert eng.model.w.layers[0].in_proj.w.shape[0] < ref.model.w.layers[0].in_proj.w.shape[0]
    got_logits = eng.prefill([eng.new_sequence(p) for p in prompts], sample=False)
    err = ((got_logits - want_logits).norm() / want_logits.norm()).item()
    assert err < 2e-3, err      # partial products are rounded before the cross-rank sum
    got_tokens = build_engine(cfg, "cpu", seed=2, max_batch=4, use_cuda_graphs=False, tp=tp).generate(prompts, 8)
    assert got_tokens == want_tokens, (got_tokens, want_tokens)
    # the all-gather + column-parallel GEMM op on its host path (tiny shapes, fp32): K shards of every rank times
    # this rank's weight rows equal the full product
    from sllm_b200.ops.core import LinearWeight
    from sllm_b200.parallel.gather import NcclGatherGemm
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(5, 64 * world, generator=gen)
    w_loc = torch.randn(24, 64 * world, generator=torch.Generator().manual_seed(20 + rank))
    res = torch.randn(5, 24, generator=gen)
    got = NcclGatherGemm(world, rank, "cpu").linear(x[:, rank * 64:(rank + 1) * 64], LinearWeight("dense", w_loc), res)
    assert torch.allclose(got, x @ w_loc.t() + res, atol=1e-4), (got - (x @ w_loc.t() + res)).abs().max()
    dist.barrier()
    if rank == 0:
        print("HYBRID_TP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

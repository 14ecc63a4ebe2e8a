"""GGUF round trips of the mixture-of-experts and the gated-delta-net hybrid families: unsharded generation equality and
shard-for-shard equality with the seeded random initialiser under tensor / expert parallelism."""
import dataclasses

import pytest
import torch

from sllm_b200.cache.paged import PagedKVCache
from sllm_b200.engine.engine import Engine
from sllm_b200.formats import gguf as G
from sllm_b200.models import family_io as FIO
from sllm_b200.models import moe as MOE
from sllm_b200.models.qwen35 import Qwen35Model, init_random_qwen35_weights, tiny_qwen35
from sllm_b200.ops.core import LinearWeight
from sllm_b200.ops.w4 import W4Weight


def _same(a, b, path=""):
    if isinstance(a, torch.Tensor):
        assert isinstance(b, torch.Tensor) and a.shape == b.shape, path
        assert torch.equal(a.float(), b.float()), path
    elif isinstance(a, LinearWeight):
        assert a.kind == b.kind, path
        _same(a.w, b.w, path + ".w")
    elif isinstance(a, W4Weight):
        assert (a.fmt, a.groups, a.n, a.k) == (b.fmt, b.groups, b.n, b.k), path
        assert torch.equal(a.tiles, b.tiles), path
        if a.tensor_scale is not None:
            assert torch.equal(a.tensor_scale, b.tensor_scale), path
    elif dataclasses.is_dataclass(a):
        for f in dataclasses.fields(a):
            _same(getattr(a, f.name), getattr(b, f.name), f"{path}.{f.name}")
    elif isinstance(a, list):
        assert len(a) == len(b), path
        for i, (x, y) in enumerate(zip(a, b)):
            _same(x, y, f"{path}[{i}]")
    else:
        assert a == b, path


def _moe_engine(cfg, w):
    m = MOE.MoeModel(cfg, w)
    return Engine(cfg, m, PagedKVCache(cfg, 64, torch.device("cpu"), kv_heads=m.local_kv_heads), "cpu", max_batch=2,
                  use_cuda_graphs=False)


@pytest.mark.parametrize("shape", ["tiny_moe", "tiny_shared_moe"])
def test_moe_round_trip_and_shards(tmp_path, shape):
    cfg = getattr(MOE, shape)()
    w = MOE.init_random_moe_weights(cfg, "cpu", seed=3)
    path = str(tmp_path / "moe.gguf")
    lock = FIO.export_family_gguf(cfg, w, path)
    g = G.verify_gguf(path, lock)
    assert g.tensors["blk.0.ffn_gate_up_exps.weight"].ttype == G.T_MXFP4
    assert g.tensors["blk.0.ffn_gate_up_exps.weight"].shape == (cfg.n_experts * 2 * cfg.expert_ffn, cfg.d_model)
    cfg2, w2 = FIO.load_family_gguf(g, "cpu")
    assert cfg2 == cfg
    _same(w, w2)
    prompt = list(range(4, 30))
    assert _moe_engine(cfg, w).generate([prompt], 5) == _moe_engine(cfg2, w2).generate([prompt], 5)
    # every rank of a 2 x 2 tensor- / expert-parallel layout reads exactly the shard the seeded initialiser keeps
    for tp_rank in range(2):
        for ep_rank in range(2):
            want = MOE.init_random_moe_weights(cfg, "cpu", seed=3, tp_size=2, tp_rank=tp_rank, ep_size=2, ep_rank=ep_rank)
            _, got = FIO.load_family_gguf(g, "cpu", tp_size=2, tp_rank=tp_rank, ep_size=2, ep_rank=ep_rank)
            _same(want, got, f"tp{tp_rank}ep{ep_rank}")
    with pytest.raises(G.GgufError):
        FIO.load_family_gguf(g, "cpu", ep_size=3)


def test_hybrid_round_trip_and_shards(tmp_path):
    from sllm_b200.cache.hybrid import HybridCache
    cfg = tiny_qwen35()
    w = init_random_qwen35_weights(cfg, "cpu", seed=5)
    path = str(tmp_path / "hy.gguf")
    lock = FIO.export_family_gguf(cfg, w, path)
    g = G.verify_gguf(path, lock)
    assert "blk.0.ssm_in.weight" in g.tensors and f"blk.{cfg.full_attention_interval - 1}.attn_q.weight" in g.tensors
    cfg2, w2 = FIO.load_family_gguf(g, "cpu")
    assert cfg2 == cfg
    _same(w, w2)

    def engine(c, ww):
        m = Qwen35Model(c, ww)
        cache = HybridCache(c, 32, torch.device("cpu"), max_seqs=6, kv_heads=m.local_kv_heads)
        return Engine(c, m, cache, "cpu", max_batch=2, use_cuda_graphs=False)

    prompt = list(range(3, 25))
    assert engine(cfg, w).generate([prompt], 5) == engine(cfg2, w2).generate([prompt], 5)
    # a geometry that divides over two ranks: every rank reads the shard the seeded initialiser keeps
    cfg.n_kv_heads, cfg.gdn_qk_heads, cfg.gdn_heads = 2, 2, 4
    path2 = str(tmp_path / "hy2.gguf")
    g2 = G.verify_gguf(path2, FIO.export_family_gguf(cfg, init_random_qwen35_weights(cfg, "cpu", seed=5), path2))
    for r in range(2):
        want = init_random_qwen35_weights(cfg, "cpu", seed=5, tp_size=2, tp_rank=r)
        _, got = FIO.load_family_gguf(g2, "cpu", tp_size=2, tp_rank=r)
        for i, (a, b) in enumerate(zip(want.layers, got.layers)):
            _same(a, b, f"rank{r}.layer{i}")


def test_llama_loader_refuses_other_families(tmp_path):
    from sllm_b200.models import loader
    cfg = MOE.tiny_moe()
    path = str(tmp_path / "m.gguf")
    lock = FIO.export_family_gguf(cfg, MOE.init_random_moe_weights(cfg, "cpu", seed=1), path)
    g = G.verify_gguf(path, lock)
    cfg2, w2, family = loader.load_model_gguf(g, "cpu")
    assert family == "moe" and type(w2).__name__ == "MoeWeights"

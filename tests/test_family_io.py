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


def test_sparse_hybrid_round_trip_and_expert_shards(tmp_path):
    """Qwen3.5-MoE layout: gated-delta-net / full-attention layers whose MLP is routed MXFP4 experts plus a gated
    shared expert.  The file round trip is bit-exact, generation is identical, and every rank of a 2 x 2 layout reads
    the shard the seeded initialiser keeps."""
    from sllm_b200.cache.hybrid import HybridCache
    from sllm_b200.models.qwen35 import tiny_qwen35_moe
    cfg = tiny_qwen35_moe()
    w = init_random_qwen35_weights(cfg, "cpu", seed=7)
    assert w.layers[0].gate_up is None and w.layers[0].router.w.shape[0] == cfg.n_experts + 8
    path = str(tmp_path / "hm.gguf")
    lock = FIO.export_family_gguf(cfg, w, path)
    g = G.verify_gguf(path, lock)
    assert g.tensors["blk.0.ffn_gate_up_exps.weight"].ttype == G.T_MXFP4 and "blk.0.ssm_in.weight" in g.tensors
    assert "blk.0.ffn_gate.weight" not in g.tensors
    cfg2, w2 = FIO.load_family_gguf(g, "cpu")
    assert cfg2 == cfg
    _same(w, w2)

    def engine(c, ww):
        m = Qwen35Model(c, ww)
        cache = HybridCache(c, 32, torch.device("cpu"), max_seqs=6, kv_heads=m.local_kv_heads)
        return Engine(c, m, cache, "cpu", max_batch=2, use_cuda_graphs=False)

    prompt = list(range(3, 25))
    out = engine(cfg, w).generate([prompt], 5)
    assert out == engine(cfg2, w2).generate([prompt], 5)
    cfg.n_kv_heads, cfg.gdn_qk_heads, cfg.gdn_heads = 2, 2, 4
    path2 = str(tmp_path / "hm2.gguf")
    g2 = G.verify_gguf(path2, FIO.export_family_gguf(cfg, init_random_qwen35_weights(cfg, "cpu", seed=7), path2))
    for tp_rank in range(2):
        for ep_rank in range(2):
            want = init_random_qwen35_weights(cfg, "cpu", seed=7, tp_size=2, tp_rank=tp_rank, ep_size=2, ep_rank=ep_rank)
            _, got = FIO.load_family_gguf(g2, "cpu", tp_size=2, tp_rank=tp_rank, ep_size=2, ep_rank=ep_rank)
            for i, (a, b) in enumerate(zip(want.layers, got.layers)):
                _same(a, b, f"tp{tp_rank}ep{ep_rank}.layer{i}")
    with pytest.raises(G.GgufError):
        FIO.load_family_gguf(g2, "cpu", ep_size=3)


def test_sparse_hybrid_mlp_matches_a_dense_evaluation():
    """One sparse MLP block of the hybrid against its definition in fp32: softmax over the selected router logits,
    the selected experts' gated MLPs on the dequantised weights, plus sigmoid(gate) x shared expert."""
    from sllm_b200.engine.batch import ForwardBatch  # noqa: F401  (the model imports it)
    from sllm_b200.models.qwen35 import tiny_qwen35_moe
    from sllm_b200 import ops
    cfg = tiny_qwen35_moe()
    cfg.weight_format = "fp32"
    w = init_random_qwen35_weights(cfg, "cpu", seed=11, std=0.2)
    m = Qwen35Model(cfg, w)
    lw = w.layers[0]
    torch.manual_seed(0)
    h = torch.randn(5, cfg.d_model)
    got = m._mlp(h.clone(), lw)
    x = ops.rmsnorm(h, lw.mlp_norm, cfg.rms_eps, cfg.norm_offset_one).float()
    logits = x @ lw.router.w.float().t()
    top = torch.topk(logits[:, :cfg.n_experts], cfg.top_k, dim=1)
    pw = torch.softmax(top.values, dim=1)
    gu_all = [torch.as_tensor(lw.exp_gate_up.dequantized(e)).float() for e in range(cfg.n_experts)]
    dn_all = [torch.as_tensor(lw.exp_down.dequantized(e)).float() for e in range(cfg.n_experts)]
    want = h.clone()
    F = cfg.expert_ffn
    for t in range(h.shape[0]):
        for j in range(cfg.top_k):
            e = int(top.indices[t, j])
            gu = gu_all[e] @ x[t]
            want[t] += pw[t, j] * (dn_all[e] @ (torch.nn.functional.silu(gu[:F]) * gu[F:]))
        sgu = lw.shared_gate_up.w.float() @ x[t]
        fs = cfg.shared_expert_ffn
        sh = lw.shared_down.w.float() @ (torch.nn.functional.silu(sgu[:fs]) * sgu[fs:])
        want[t] += torch.sigmoid(logits[t, cfg.n_experts]) * sh
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2)


def _hf_qwen35_checkpoint(root, cfg, w):
    """Writes `w` under the tensor names and layouts of a Qwen3.5 Hugging Face checkpoint (query and output gate
    packed per head, the gated-delta-net input projection split in four, experts as packed U8 + E8M0 planes), plus a
    vision and a multi-token-prediction tensor the decoder does not consume."""
    import json
    from safetensors.torch import save_file
    t = {}
    hq, hd, d = cfg.n_heads, cfg.head_dim, cfg.d_model
    ghd, vh, qh = cfg.gdn_head_dim, cfg.gdn_heads, cfg.gdn_qk_heads
    width = (2 * qh + vh) * ghd
    q, kv, f = cfg.q_size, cfg.kv_size, cfg.ffn
    for i, l in enumerate(w.layers):
        p = f"model.language_model.layers.{i}."
        t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"] = l.in_norm, l.mlp_norm
        if l.router is not None:
            E, F = cfg.n_experts, cfg.expert_ffn
            t[p + "mlp.gate.weight"] = l.router.w[:E]
            t[p + "mlp.shared_expert_gate.weight"] = l.router.w[E:E + 1]
            fs = cfg.shared_expert_ffn
            t[p + "mlp.shared_expert.gate_proj.weight"], t[p + "mlp.shared_expert.up_proj.weight"] = l.shared_gate_up.w[:fs], l.shared_gate_up.w[fs:]
            t[p + "mlp.shared_expert.down_proj.weight"] = l.shared_down.w
            for e in range(E):
                pk, sc = l.exp_gate_up.to_file_layout(e)
                for j, stem in enumerate(("gate_proj", "up_proj")):
                    t[f"{p}mlp.experts.{e}.{stem}.weight"] = torch.from_numpy(pk[j * F:(j + 1) * F].copy())
                    t[f"{p}mlp.experts.{e}.{stem}.weight_scale"] = torch.from_numpy(sc[j * F:(j + 1) * F].copy())
                pk, sc = l.exp_down.to_file_layout(e)
                t[f"{p}mlp.experts.{e}.down_proj.weight"] = torch.from_numpy(pk.copy())
                t[f"{p}mlp.experts.{e}.down_proj.weight_scale"] = torch.from_numpy(sc.copy())
        else:
            t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"], t[p + "mlp.down_proj.weight"] = l.gate_up.w[:f], l.gate_up.w[f:], l.down.w
        if l.kind == "full":
            a = p + "self_attn."
            packed = torch.stack([l.qkv.w[:q].view(hq, hd, d), l.gate.w.view(hq, hd, d)], dim=1).reshape(2 * q, d)
            t[a + "q_proj.weight"], t[a + "k_proj.weight"], t[a + "v_proj.weight"] = packed, l.qkv.w[q:q + kv], l.qkv.w[q + kv:]
            t[a + "o_proj.weight"], t[a + "q_norm.weight"], t[a + "k_norm.weight"] = l.o.w, l.q_norm, l.k_norm
        else:
            a = p + "linear_attn."
            wi = l.in_proj.w
            t[a + "in_proj_qkv.weight"], t[a + "in_proj_z.weight"] = wi[:width], wi[width:width + vh * ghd]
            t[a + "in_proj_b.weight"] = wi[width + vh * ghd:width + vh * ghd + vh]
            t[a + "in_proj_a.weight"] = wi[width + vh * ghd + vh:width + vh * ghd + 2 * vh]
            t[a + "conv1d.weight"] = l.conv_w.view(width, 1, cfg.gdn_conv_kernel)
            t[a + "A_log"], t[a + "dt_bias"], t[a + "norm.weight"], t[a + "out_proj.weight"] = l.a_log, l.dt_bias, l.out_norm, l.out_proj.w
    t["model.language_model.embed_tokens.weight"], t["model.language_model.norm.weight"] = w.embed, w.final_norm
    t["lm_head.weight"] = w.lm_head.w
    t["model.visual.blocks.0.norm1.weight"] = torch.ones(8, dtype=torch.bfloat16)
    t["mtp.norm.weight"] = torch.ones(8, dtype=torch.bfloat16)
    save_file({k: v.contiguous().clone() for k, v in t.items()}, str(root / "model.safetensors"))
    text = {"model_type": "qwen3_5_moe_text" if cfg.n_experts else "qwen3_5_text", "hidden_size": d,
            "num_hidden_layers": cfg.n_layers, "num_attention_heads": hq, "num_key_value_heads": cfg.n_kv_heads, "head_dim": hd,
            "intermediate_size": f, "vocab_size": cfg.vocab, "full_attention_interval": cfg.full_attention_interval,
            "linear_num_value_heads": vh, "linear_num_key_heads": qh, "linear_key_head_dim": ghd, "linear_value_head_dim": ghd,
            "linear_conv_kernel_dim": cfg.gdn_conv_kernel, "rms_norm_eps": cfg.rms_eps, "attn_output_gate": True,
            "max_position_embeddings": cfg.max_context,
            "rope_parameters": {"rope_theta": cfg.rope_theta, "partial_rotary_factor": cfg.rotary_dim / hd}}
    if cfg.n_experts:
        text.update(num_experts=cfg.n_experts, num_experts_per_tok=cfg.top_k, moe_intermediate_size=cfg.expert_ffn,
                    shared_expert_intermediate_size=cfg.shared_expert_ffn)
    (root / "config.json").write_text(json.dumps({"text_config": text, "tie_word_embeddings": False, "_name_or_path": cfg.name}))


@pytest.mark.parametrize("sparse", [False, True])
def test_hf_qwen35_importer(tmp_path, capsys, sparse):
    """`sllm-convert-gguf --kind hf-qwen35` on a synthetic checkpoint in the source layout: every decoder tensor lands
    where the seeded weights had it, vision / MTP tensors are recorded as known-unconsumed, an unknown tensor is refused."""
    import json
    from sllm_b200.cli import convert
    from sllm_b200.formats import model_lock as ML
    from sllm_b200.models.qwen35 import tiny_qwen35_moe
    cfg = tiny_qwen35_moe() if sparse else tiny_qwen35()
    w = init_random_qwen35_weights(cfg, "cpu", seed=9)
    src = tmp_path / "src"
    src.mkdir()
    _hf_qwen35_checkpoint(src, cfg, w)
    lock = ML.make_model_lock(str(src), "local/tiny-q35", "0" * 40, ["tiny-q35"], {"family": "qwen35"}, {"kind": "none"})
    (tmp_path / "lock.json").write_text(json.dumps(lock))
    out, dl = str(tmp_path / "m.gguf"), str(tmp_path / "m.lock.json")
    rc = convert.main(["--kind", "hf-qwen35", "--lock", str(tmp_path / "lock.json"), "--cache", str(src), "--output", out,
                       "--derived-lock", dl])
    assert rc == 0
    event = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert event["written"] and event["known_unconsumed_tensors"] == 2 and event["source_lock_fingerprints"] == [lock["fingerprint"]]
    g = G.verify_gguf(out, G.read_derived_lock(dl))
    assert g.recipe()["known_unconsumed_tensors"] == ["model.visual.blocks.0.norm1.weight", "mtp.norm.weight"]
    cfg2, w2 = FIO.load_family_gguf(g, "cpu")
    for k in ("n_layers", "d_model", "head_dim", "rotary_dim", "gdn_heads", "n_experts", "top_k", "shared_expert_ffn", "rope_theta"):
        assert getattr(cfg2, k) == getattr(cfg, k), k
    _same(w.layers, w2.layers, "layers")
    _same(w.embed, w2.embed)
    _same(w.lm_head, w2.lm_head)
    # an extra tensor outside the known components is refused
    from safetensors.torch import load_file, save_file
    t = load_file(str(src / "model.safetensors"))
    t["model.language_model.layers.0.surprise.weight"] = torch.ones(4)
    save_file(t, str(src / "model.safetensors"))
    lock = ML.make_model_lock(str(src), "local/tiny-q35", "0" * 40, ["tiny-q35"], {"family": "qwen35"}, {"kind": "none"})
    (tmp_path / "lock.json").write_text(json.dumps(lock))
    assert convert.main(["--kind", "hf-qwen35", "--lock", str(tmp_path / "lock.json"), "--cache", str(src), "--output", out,
                         "--derived-lock", dl]) != 0
    assert "unconsumed tensors" in capsys.readouterr().out


def test_hybrid_family_with_fp8_projections(tmp_path):
    """Block-scaled FP8 projections in the hybrid family: the model runs (logits near the bf16 model's), the GGUF round
    trip is bit-exact, and tensor-parallel ranks read the shard the seeded initialiser keeps (row shards and 128-column
    aligned column shards of values and block scales)."""
    from sllm_b200.cache.hybrid import HybridCache
    cfg = tiny_qwen35()
    cfg.weight_format = "fp8"
    w = init_random_qwen35_weights(cfg, "cpu", seed=5)
    assert w.layers[0].in_proj.kind == "fp8" and w.layers[3].qkv.kind == "fp8" and w.layers[0].gate_up.kind == "fp8"
    path = str(tmp_path / "hy8.gguf")
    g = G.verify_gguf(path, FIO.export_family_gguf(cfg, w, path))
    assert g.tensors["blk.0.ssm_in.weight"].ttype == G.T_I8 and "blk.0.ssm_in.weight.scale" in g.tensors
    cfg2, w2 = FIO.load_family_gguf(g, "cpu")
    assert cfg2 == cfg

    def same_lin(a, b, path):
        assert a.kind == b.kind == "fp8", path
        assert torch.equal(a.w, b.w) and torch.equal(a.scale_t, b.scale_t), path

    for i, (a, b) in enumerate(zip(w.layers, w2.layers)):
        for name in ("gate_up", "down", "qkv", "gate", "o", "in_proj", "out_proj"):
            if getattr(a, name) is not None:
                same_lin(getattr(a, name), getattr(b, name), f"layer{i}.{name}")

    def engine(c, ww):
        m = Qwen35Model(c, ww)
        cache = HybridCache(c, 32, torch.device("cpu"), max_seqs=6, kv_heads=m.local_kv_heads)
        return Engine(c, m, cache, "cpu", max_batch=2, use_cuda_graphs=False)

    prompt = list(range(3, 25))
    e8 = engine(cfg, w)
    assert e8.generate([prompt], 5) == engine(cfg2, w2).generate([prompt], 5)
    cfg16 = tiny_qwen35()
    e16 = engine(cfg16, init_random_qwen35_weights(cfg16, "cpu", seed=5))
    l8 = e8.prefill([e8.new_sequence(prompt)], sample=False).float()
    l16 = e16.prefill([e16.new_sequence(prompt)], sample=False).float()
    assert ((l8 - l16).norm() / l16.norm()).item() < 0.15
    # shards: a geometry that divides over two ranks with 128-aligned column shards
    cfg.n_kv_heads, cfg.gdn_qk_heads, cfg.gdn_heads, cfg.head_dim, cfg.rotary_dim = 2, 2, 4, 128, 32
    path2 = str(tmp_path / "hy8b.gguf")
    g2 = G.verify_gguf(path2, FIO.export_family_gguf(cfg, init_random_qwen35_weights(cfg, "cpu", seed=5), path2))
    for r in range(2):
        want = init_random_qwen35_weights(cfg, "cpu", seed=5, tp_size=2, tp_rank=r)
        _, got = FIO.load_family_gguf(g2, "cpu", tp_size=2, tp_rank=r)
        for i, (a, b) in enumerate(zip(want.layers, got.layers)):
            for name in ("gate_up", "qkv", "gate", "in_proj"):            # row shards: quantisation is per row block
                if getattr(a, name) is not None:
                    same_lin(getattr(a, name), getattr(b, name), f"rank{r}.layer{i}.{name}")
            for name in ("down", "o", "out_proj"):                         # column shards: whole 128-column blocks
                if getattr(a, name) is not None:
                    same_lin(getattr(a, name), getattr(b, name), f"rank{r}.layer{i}.{name}")


def test_converter_writes_fp8_hybrid_files(tmp_path, capsys):
    from sllm_b200.cli import convert
    from sllm_b200.models import loader
    out, dl = str(tmp_path / "q8.gguf"), str(tmp_path / "q8.lock.json")
    assert convert.main(["--kind", "random-llama", "--artifact", "tiny-qwen35", "--weight-format", "fp8", "--output", out,
                         "--derived-lock", dl]) == 0
    capsys.readouterr()
    g = G.verify_gguf(out, G.read_derived_lock(dl))
    cfg, w, family = loader.load_model_gguf(g, "cpu")
    assert family == "qwen35" and cfg.weight_format == "fp8" and w.layers[0].in_proj.kind == "fp8"
    assert convert.main(["--kind", "random-llama", "--artifact", "tiny-moe", "--weight-format", "fp8", "--output", out,
                         "--derived-lock", dl]) != 0

"""Model families beyond the plain dense decoder, on the CPU oracle path: the gated-delta-net hybrid and the
Gemma-style options (q/k norm, sandwich norms, gelu-tanh, soft-cap, scaled tied embeddings, window schedule)."""
import pytest
import torch

from sllm_b200.engine.engine import build_engine
from sllm_b200.models import config as MC
from sllm_b200.models.qwen35 import tiny_qwen35


def test_hybrid_decode_equals_prefill_and_state_slots_are_isolated():
    cfg = tiny_qwen35()
    cfg.weight_format, cfg.kv_format = "fp32", "fp32"
    eng = build_engine(cfg, "cpu", seed=1, num_pages=32, max_batch=2, use_cuda_graphs=False)
    p = [list(range(3, 20)), [5, 6, 7]]
    both = eng.generate(p, 6)
    alone = [eng.generate([x], 6)[0] for x in p]
    assert both == alone                                     # batch rows do not leak state into one another
    assert eng.generate([p[0] + both[0][:3]], 3)[0] == both[0][3:]
    assert len(eng.cache.slot_of) == 0 and len(eng.cache._free) == eng.cache.max_seqs
    # chunked prefill carries the conv window and the recurrent matrix across chunks
    s = eng.new_sequence(p[0])
    t_chunked = eng.prefill([s], chunk_tokens=5)[0]
    eng.free_sequence(s)
    assert t_chunked == both[0][0]
    # a recurrent state can be shared only at the end of the source's computed tokens
    src = eng.new_sequence(p[0])
    eng.prefill([src])
    f1 = eng.fork_sequence(src, p[0] + [9, 9])
    assert f1.num_computed == len(p[0])
    f2 = eng.fork_sequence(src, p[0][:10] + [1, 2])
    assert f2.num_computed == 0
    a = eng.prefill([f1])[0]
    fresh = eng.new_sequence(p[0] + [9, 9])
    assert eng.prefill([fresh])[0] == a
    with pytest.raises(ValueError):
        eng.rollback(src, 3)
    for q in (src, f1, f2, fresh):
        eng.free_sequence(q)


def test_gemma_style_options():
    cfg = MC.ModelConfig(name="tiny-gemma", family="gemma4", n_layers=3, d_model=128, n_heads=4, n_kv_heads=2, head_dim=32, ffn=256,
                         vocab=512, act="gelu_tanh", tie_embeddings=True, embedding_scale=128 ** 0.5, logit_softcap=30.0,
                         weight_format="fp32", kv_format="fp32", sliding_window=8, window_layers=[True, True, False], qk_norm=True,
                         post_norms=True, max_context=128)
    eng = build_engine(cfg, "cpu", seed=2, num_pages=32, max_batch=2, use_cuda_graphs=False)
    assert eng.model.w.lm_head.w is eng.model.w.embed                       # tied
    prompt = list(range(7, 40))
    out = eng.generate([prompt], 8)[0]
    assert eng.generate([prompt + out[:4]], 4)[0] == out[4:]                 # window + cache consistent across decode
    s = eng.new_sequence(prompt)
    lg = eng.prefill([s], sample=False)
    eng.free_sequence(s)
    assert lg.abs().max() <= 30.0 + 1e-4                                      # soft-capped
    # the options matter: switching them off changes the logits
    import dataclasses
    plain = dataclasses.replace(cfg, post_norms=False, qk_norm=False, logit_softcap=0.0)
    e2 = build_engine(plain, "cpu", seed=2, num_pages=32, max_batch=2, use_cuda_graphs=False)
    s = e2.new_sequence(prompt)
    assert not torch.allclose(e2.prefill([s], sample=False), lg, atol=1e-3)
    assert MC.NAMED["gemma4"]().window_layers[:6] == [True] * 5 + [False]
    assert MC.NAMED["qwen35-hybrid"]().full_attention_interval == 4


def test_gemma4_attention_details(tmp_path):
    """Proportional rotary layout on the full layers, own rotary base on the sliding layers, unweighted value norm,
    softmax scale 1, per-layer output scalar, full layers without a value projection; and their GGUF round trip."""
    import dataclasses
    from sllm_b200.ops import reference as ref
    # the pair layout itself, against a direct restatement (reference: crates/sllm-core/src/op.rs:805-811)
    torch.manual_seed(0)
    x = torch.randn(5, 3, 32)
    pos = torch.tensor([0, 1, 7, 19, 40], dtype=torch.int32)
    y = ref.rope_split_half(x, pos, 1e6, rotary_dim=8, pair_offset=16)
    for i in range(32):
        if i < 4 or 16 <= i < 20:
            f = i if i < 4 else i - 16
            ang = pos.float() * (1e6 ** (-2.0 * f / 32))
            a, b = x[:, :, f], x[:, :, f + 16]
            want = a * ang.cos()[:, None] - b * ang.sin()[:, None] if i < 4 else b * ang.cos()[:, None] + a * ang.sin()[:, None]
            assert torch.allclose(y[:, :, i], want, atol=1e-5)
        else:
            assert torch.equal(y[:, :, i], x[:, :, i])
    cfg = MC.ModelConfig(name="tiny-gemma4", family="gemma4", n_layers=3, d_model=128, n_heads=4, n_kv_heads=2, head_dim=32,
                         ffn=256, vocab=512, act="gelu_tanh", tie_embeddings=True, embedding_scale=128 ** 0.5,
                         logit_softcap=30.0, weight_format="fp32", kv_format="fp32", sliding_window=8,
                         window_layers=[True, True, False], qk_norm=True, post_norms=True, max_context=128,
                         rope_theta=1e6, rope_theta_local=1e4, rope_proportional=True, rotary_dim_full=8, v_norm=True,
                         attn_scale=1.0, layer_scalar=True, k_equals_v_full=True)
    assert cfg.layer_rope(0) == (1e4, 32, 0) and cfg.layer_rope(2) == (1e6, 8, 16)
    eng = build_engine(cfg, "cpu", seed=2, num_pages=32, max_batch=2, use_cuda_graphs=False)
    full = eng.model.w.layers[2].qkv.w
    assert torch.equal(full[128:192], full[192:256]) and not torch.equal(eng.model.w.layers[0].qkv.w[128:192],
                                                                          eng.model.w.layers[0].qkv.w[192:256])
    for i, l in enumerate(eng.model.w.layers):
        l.layer_scalar.fill_(0.5 + 0.25 * i)
    prompt = list(range(7, 40))
    out = eng.generate([prompt], 8)[0]
    assert eng.generate([prompt + out[:4]], 4)[0] == out[4:]
    s = eng.new_sequence(prompt)
    lg = eng.prefill([s], sample=False)
    eng.free_sequence(s)
    for off in ({"v_norm": False}, {"attn_scale": None}, {"rope_proportional": False}, {"rope_theta_local": 0.0}):
        e2 = build_engine(dataclasses.replace(cfg, **off), "cpu", seed=2, num_pages=32, max_batch=2, use_cuda_graphs=False)
        for i, l in enumerate(e2.model.w.layers):
            l.layer_scalar.fill_(0.5 + 0.25 * i)
        s = e2.new_sequence(prompt)
        assert not torch.allclose(e2.prefill([s], sample=False), lg, atol=1e-4), off
    # the file keeps the per-layer vectors and the scalar
    from sllm_b200.formats import gguf as G
    from sllm_b200.models.loader import export_llama_gguf, load_llama_gguf
    path = str(tmp_path / "g4.gguf")
    export_llama_gguf(cfg, eng.model.w, path)
    cfg2, w2 = load_llama_gguf(G.GgufFile(path), "cpu")
    assert cfg2 == cfg
    assert [float(l.layer_scalar) for l in w2.layers] == [0.5, 0.75, 1.0]
    assert w2.layers[1].q_norm is not None and w2.layers[1].post_mlp_norm is not None
    from sllm_b200.cache.paged import PagedKVCache
    from sllm_b200.engine.engine import Engine
    from sllm_b200.models.llama import LlamaModel
    m3 = LlamaModel(cfg2, w2, None)
    e3 = Engine(cfg2, m3, PagedKVCache(cfg2, 32, torch.device("cpu"), kv_heads=m3.local_kv_heads), torch.device("cpu"),
                max_batch=2, use_cuda_graphs=False)
    assert e3.generate([prompt], 8)[0] == out


def test_hybrid_family_tensor_parallel_cpu():
    """Two gloo ranks with sharded heads reproduce the single-rank hybrid model."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29843", os.path.join(here, "hybrid_tp_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and "HYBRID_TP_OK" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-3000:]

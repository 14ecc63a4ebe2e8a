"""Mixture-of-experts: routing / permutation oracles, the tiny MoE model on CPU, expert-parallel equivalence."""
import numpy as np
import pytest
import torch

from sllm_b200.cache.paged import PagedKVCache
from sllm_b200.engine.engine import Engine
from sllm_b200.models import moe as MOE
from sllm_b200.ops import moe as M


def test_route_and_permute_cpu():
    torch.manual_seed(0)
    logits = torch.randn(7, 8)
    logits[0, 3] = logits[0, 5] = 9.0               # tie: the lower index wins first
    logits[1, 2] = float("nan")
    idx, w = M.route(logits, 2)
    assert idx[0].tolist() == [3, 5] and 2 not in idx[1].tolist()
    assert torch.allclose(w.sum(1), torch.ones(7), atol=1e-6)
    idx_all, w_all = M.route(logits, 2, softmax_all=True)
    assert torch.equal(idx_all, idx) and (w_all.sum(1) < 1).all()
    tok_off, src, dst, pw = M.permute(idx, w, 2, 6)
    n = int(tok_off[-1])
    assert n == int(((idx >= 2) & (idx < 6)).sum())
    for t in range(7):
        for j in range(2):
            p = int(dst[t, j])
            e = int(idx[t, j])
            if 2 <= e < 6:
                assert int(src[p]) == t and float(pw[p]) == float(w[t, j])
                assert int(tok_off[e - 2]) <= p < int(tok_off[e - 1])
            else:
                assert p == -1
    x = torch.randn(7, 16)
    xp = M.gather(x, src, tok_off)
    assert torch.equal(xp[:n], x[src[:n].long()])
    y = M.combine(xp * 1.0, dst, x)
    want = x.clone()
    for t in range(7):
        for j in range(2):
            if dst[t, j] >= 0:
                want[t] += x[t]
    assert torch.allclose(y, want)


def _engine(cfg, ep=None, ep_size=1, ep_rank=0):
    w = MOE.init_random_moe_weights(cfg, "cpu", seed=2, ep_size=ep_size, ep_rank=ep_rank)
    model = MOE.MoeModel(cfg, w, ep=ep)
    cache = PagedKVCache(cfg, 64, torch.device("cpu"), kv_heads=model.local_kv_heads)
    return Engine(cfg, model, cache, "cpu", max_batch=4, use_cuda_graphs=False)


def test_tiny_moe_generates_and_matches_dense_reference():
    cfg = MOE.tiny_moe()
    cfg.weight_format, cfg.kv_format = "fp32", "fp32"
    eng = _engine(cfg)
    prompts = [list(range(5, 30)), [7, 8, 9]]
    out = eng.generate(prompts, 6)
    assert len(out) == 2 and all(len(o) == 6 for o in out)
    # decode equals prefill of the extended prompt (KV cache, window and sinks consistent)
    again = eng.generate([prompts[0] + out[0][:3]], 3)[0]
    assert again == out[0][3:6]
    # one MoE block against a dense restatement: every expert on every token, masked by the routing weights
    lw = eng.model.w.layers[0]
    x = torch.randn(5, cfg.d_model)
    logits = x @ lw.router.w.float().t()
    idx, rw = M.route(logits, cfg.top_k)
    yp, dst = M.experts_forward(x, idx, rw, lw.gate_up, lw.down, cfg.act, 0, cfg.n_experts)
    got = M.combine(yp, dst, None)
    want = torch.zeros(5, cfg.d_model)
    for t in range(5):
        for j in range(cfg.top_k):
            e = int(idx[t, j])
            gu = x[t] @ lw.gate_up.dequantized(e).t()
            g, u = gu[:cfg.expert_ffn], gu[cfg.expert_ffn:]
            want[t] += float(rw[t, j]) * ((torch.nn.functional.silu(g) * u) @ lw.down.dequantized(e).t())
    assert torch.allclose(got, want, rtol=2e-3, atol=2e-4)


def test_expert_parallel_partials_add_up():
    """Two expert-parallel ranks, emulated in one process: the sum of their partial outputs is the full MoE output."""
    cfg = MOE.tiny_moe()
    cfg.weight_format, cfg.kv_format = "fp32", "fp32"
    full = MOE.init_random_moe_weights(cfg, "cpu", seed=2).layers[0]
    parts = [MOE.init_random_moe_weights(cfg, "cpu", seed=2, ep_size=2, ep_rank=r).layers[0] for r in range(2)]
    x = torch.randn(6, cfg.d_model)
    idx, rw = M.route(x @ full.router.w.float().t(), cfg.top_k)
    yp, dst = M.experts_forward(x, idx, rw, full.gate_up, full.down, cfg.act, 0, 8)
    want = M.combine(yp, dst, None)
    acc = torch.zeros_like(want)
    for r in range(2):
        yp_r, dst_r = M.experts_forward(x, idx, rw, parts[r].gate_up, parts[r].down, cfg.act, r * 4, r * 4 + 4)
        acc += M.combine(yp_r, dst_r, None)
    assert torch.allclose(acc, want, rtol=1e-5, atol=1e-6)


def test_shared_expert_and_256_way_routing():
    """Qwen3.5-MoE layer: top-8 of 256 experts plus a dense shared expert under a per-token sigmoid gate
    (reference: native/hip/src/moe_expert_kernel.hip.cpp:134-174)."""
    cfg = MOE.tiny_shared_moe()
    cfg.weight_format, cfg.kv_format = "fp32", "fp32"
    eng = _engine(cfg)
    lw = eng.model.w.layers[0]
    assert lw.router.w.shape[0] == cfg.n_experts + 8 and lw.shared_gate_up.w.shape == (2 * cfg.shared_expert_ffn, cfg.d_model)
    prompts = [list(range(5, 30)), [7, 8, 9]]
    out = eng.generate(prompts, 5)
    assert eng.generate([prompts[0] + out[0][:2]], 3)[0] == out[0][2:5]
    # one block against a direct restatement
    torch.manual_seed(1)
    x = torch.randn(4, cfg.d_model)
    logits = x @ lw.router.w.float().t()
    idx, rw = M.route(logits[:, :cfg.n_experts], cfg.top_k)
    assert idx.shape == (4, 8) and int(idx.max()) < 256
    yp, dst = M.experts_forward(x, idx, rw, lw.gate_up, lw.down, cfg.act, 0, cfg.n_experts)
    routed = M.combine(yp, dst, None)
    gu = x @ lw.shared_gate_up.w.float().t()
    fs = cfg.shared_expert_ffn
    sh = (torch.nn.functional.silu(gu[:, :fs]) * gu[:, fs:]) @ lw.shared_down.w.float().t()
    want = routed + torch.sigmoid(x @ lw.router.w.float()[cfg.n_experts]).unsqueeze(1) * sh
    got = M.shared_add(routed, sh, logits[:, cfg.n_experts])
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5)
    from sllm_b200.models import config as MC
    big = MC.NAMED["qwen35-moe"]()
    assert (big.n_experts, big.top_k, big.shared_expert_ffn) == (256, 8, 512)

"""Independent NumPy restatement of a Llama-style decoder (fp32, dense causal attention, no paging,
no KV cache reuse): the CPU reference path for token-for-token checks of the engine.

It deliberately imports nothing from the implementation (ops, models, cache); weights are passed as
plain arrays.  The reference ships only tiny NumPy oracles for individual ops
(tests/reference/oracles.py:22-142) and a fake backend that never computes (crates/sllm-core/src/fake.rs:8),
so a whole-model oracle is restated here from the layer order in crates/sllm-core/src/qwen_graph.rs:2524-3501.
"""
from __future__ import annotations

import numpy as np


def rmsnorm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def rope(x, pos, theta):
    """x: [T, H, D]; split-half rotation: channel i pairs with i + D/2."""
    t, h, d = x.shape
    half = d // 2
    inv = theta ** (-2.0 * np.arange(half, dtype=np.float32) / d)
    ang = pos[:, None].astype(np.float32) * inv[None, :]
    cs, sn = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * cs - b * sn, b * cs + a * sn], axis=-1)


def forward_logits(weights: dict, cfg: dict, tokens: np.ndarray) -> np.ndarray:
    """Logits [T, vocab] for one sequence of token ids (recomputed from scratch)."""
    t = len(tokens)
    hq, hkv, hd = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    g = hq // hkv
    pos = np.arange(t)
    h = weights["embed"][tokens].astype(np.float32)
    mask = np.triu(np.ones((t, t), dtype=bool), 1)
    for lw in weights["layers"]:
        x = rmsnorm(h, lw["attn_norm"], cfg["rms_eps"])
        qkv = x @ lw["qkv"].T
        q = rope(qkv[:, :hq * hd].reshape(t, hq, hd), pos, cfg["rope_theta"])
        k = rope(qkv[:, hq * hd:(hq + hkv) * hd].reshape(t, hkv, hd), pos, cfg["rope_theta"])
        v = qkv[:, (hq + hkv) * hd:].reshape(t, hkv, hd)
        k, v = np.repeat(k, g, axis=1), np.repeat(v, g, axis=1)
        s = np.einsum("qhd,khd->hqk", q, k) / np.sqrt(hd)
        s = np.where(mask[None], -np.inf, s)
        s = s - s.max(-1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(-1, keepdims=True)
        a = np.einsum("hqk,khd->qhd", p, v).reshape(t, hq * hd)
        h = h + a @ lw["o"].T
        x = rmsnorm(h, lw["mlp_norm"], cfg["rms_eps"])
        gu = x @ lw["gate_up"].T
        ffn = gu.shape[1] // 2
        gate, up = gu[:, :ffn], gu[:, ffn:]
        h = h + (gate / (1.0 + np.exp(-gate)) * up) @ lw["down"].T
    x = rmsnorm(h, weights["final_norm"], cfg["rms_eps"])
    return x @ weights["lm_head"].T


def greedy_generate(weights: dict, cfg: dict, prompt: list, n_new: int):
    """Returns (generated token ids, logits of each generation step)."""
    toks = list(prompt)
    out, step_logits = [], []
    for _ in range(n_new):
        lg = forward_logits(weights, cfg, np.asarray(toks))[-1]
        nxt = int(np.argmax(lg))
        out.append(nxt)
        step_logits.append(lg)
        toks.append(nxt)
    return out, step_logits

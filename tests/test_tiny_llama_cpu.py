"""Config 1: tiny Llama-style decoder on CPU, engine (paged KV, incremental decode) vs the independent
NumPy oracle (dense attention recomputed from scratch), token for token."""
import numpy as np
import torch

from sllm_b200.engine.engine import build_engine
from sllm_b200.models.config import tiny_llama
from sllm_b200.oracle import tiny_llama as oracle


def _np_weights(w):
    return {
        "embed": w.embed.numpy(), "final_norm": w.final_norm.numpy(), "lm_head": w.lm_head.w.numpy(),
        "layers": [{"attn_norm": l.attn_norm.numpy(), "qkv": l.qkv.w.numpy(), "o": l.o.w.numpy(),
                    "mlp_norm": l.mlp_norm.numpy(), "gate_up": l.gate_up.w.numpy(), "down": l.down.w.numpy()}
                   for l in w.layers],
    }


def test_tiny_llama_greedy_matches_oracle():
    cfg = tiny_llama()
    cfg.max_context = 128
    eng = build_engine(cfg, "cpu", seed=0, max_batch=2, use_cuda_graphs=False)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (16,), generator=g).tolist(),
               torch.randint(0, cfg.vocab, (32,), generator=g).tolist()]
    got = eng.generate(prompts, 32)
    w = _np_weights(eng.model.w)
    c = cfg.to_dict()
    for p, toks in zip(prompts, got):
        want, _ = oracle.greedy_generate(w, c, p, 32)
        assert toks == want


def test_tiny_llama_logits_close_to_oracle():
    cfg = tiny_llama()
    cfg.max_context = 64
    eng = build_engine(cfg, "cpu", seed=0, max_batch=2, use_cuda_graphs=False)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab, (16,), generator=g).tolist(),
               torch.randint(0, cfg.vocab, (32,), generator=g).tolist()]
    seqs = [eng.new_sequence(p) for p in prompts]
    lg = eng.prefill(seqs, sample=False).numpy()
    w = _np_weights(eng.model.w)
    for i, p in enumerate(prompts):
        want = oracle.forward_logits(w, cfg.to_dict(), np.asarray(p))[-1]
        assert np.abs(lg[i] - want).max() < 2e-4 * max(1.0, np.abs(want).max())
    # chunked prefill gives the same logits
    seqs2 = [eng.new_sequence(p) for p in prompts]
    lg2 = eng.prefill(seqs2, chunk_tokens=7, sample=False).numpy()
    assert np.abs(lg2 - lg).max() < 1e-4

"""Accuracy runner: how far a quantised configuration moves the next-token distribution of the SAME model.

    python -m sllm_b200.evidence.accuracy --candidate nvfp4 [--act4] [--baseline bf16] [--device cuda|cpu]

Two engines are built from one seed - the seeded initialiser draws the same bf16 values for every weight format and
then quantises them - and run over the same prompts; the report (schema ``sllm-accuracy-v1``) gives, per configuration
pair, the mean and maximum Kullback-Leibler divergence KL(baseline || candidate) of the next-token distributions (fp64),
the top-1 agreement and the relative error of the logits.  Candidates: ``fp8`` (block-scaled E4M3 weights + FP8
activations), ``nvfp4`` / ``mxfp4`` (4-bit weights, bf16 activations), and the same with ``--act4`` (4-bit activations
on the block-scaled tensor-core kernel).  Runs on a GPU through the kernels, or on the CPU through their oracles.

Reference: the accuracy runners among crates/sllm-hip/src/bin/ (FP8 / NVFP4 KLD evidence).
"""
from __future__ import annotations

import argparse
import json
import sys

SCHEMA = "sllm-accuracy-v1"


def _logits(cfg, device: str, prompts: list, act4: bool):
    import torch
    from ..engine.engine import build_engine
    from ..ops import w4
    w4.set_w4a4(act4)
    try:
        eng = build_engine(cfg, device, seed=7, num_pages=64, max_batch=4, use_cuda_graphs=False)
        rows = []
        for p in prompts:
            s = eng.new_sequence(p)
            rows.append(eng.prefill([s], sample=False).double().cpu()[0])
            eng.free_sequence(s)
        return torch.stack(rows)
    finally:
        w4.set_w4a4(False)


def compare(baseline: str = "bf16", candidate: str = "fp8", act4: bool = False, device: str = "cpu", layers: int = 2,
            prompts: int = 8, prompt_len: int = 24) -> dict:
    """Builds the two engines and returns the report.  Prompts of at most 32 tokens keep a `--act4` candidate on its
    4-bit path (longer batches of rows keep bf16 activations by design)."""
    import torch
    from ..models import config as MC
    if act4 and candidate not in ("nvfp4", "mxfp4"):
        raise ValueError("--act4 applies to the 4-bit weight formats")
    if act4 and prompt_len > 32:
        raise ValueError("a 4-bit-activation candidate is measured on prompts of at most 32 tokens")

    def cfg(fmt):
        return MC.ModelConfig(name="accuracy", n_layers=layers, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024,
                              vocab=2048, weight_format=fmt, kv_format="bf16", max_context=256)

    g = torch.Generator().manual_seed(11)
    ps = [torch.randint(3, 2048, (prompt_len,), generator=g).tolist() for _ in range(prompts)]
    lb = _logits(cfg(baseline), device, ps, False)
    lc = _logits(cfg(candidate), device, ps, act4)
    pb, pc = torch.log_softmax(lb, dim=-1), torch.log_softmax(lc, dim=-1)
    kl = (pb.exp() * (pb - pc)).sum(dim=-1)
    return {"schema": SCHEMA, "device": device, "baseline": baseline, "candidate": candidate + ("+act4" if act4 else ""),
            "model": {"layers": layers, "d_model": 512, "vocab": 2048, "weights": "seeded random, shared by both"},
            "prompts": prompts, "prompt_len": prompt_len,
            "kl_mean": float(kl.mean()), "kl_max": float(kl.max()),
            "top1_agreement": float((lb.argmax(-1) == lc.argmax(-1)).double().mean()),
            "logit_rel_err": float((lb - lc).norm() / (lb.norm() + 1e-30)), "finite": bool(torch.isfinite(lc).all())}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m sllm_b200.evidence.accuracy")
    ap.add_argument("--baseline", default="bf16", choices=("bf16", "fp8", "nvfp4", "mxfp4"))
    ap.add_argument("--candidate", default="fp8", choices=("bf16", "fp8", "nvfp4", "mxfp4"))
    ap.add_argument("--act4", action="store_true")
    ap.add_argument("--device", default=None, choices=("cpu", "cuda"))
    ap.add_argument("--layers", type=int, default=2)
    a = ap.parse_args(argv)
    import torch
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    if dev == "cuda" and not torch.cuda.is_available():
        print(json.dumps({"schema": SCHEMA, "executed": False, "unavailable": "no CUDA device"}))
        return 0
    rep = compare(a.baseline, a.candidate, a.act4, dev, a.layers)
    print(json.dumps(rep, sort_keys=True))
    return 0 if rep["finite"] else 1


if __name__ == "__main__":
    sys.exit(main())

"""Gated-delta-net ops (causal conv + SiLU with rolling state, gated delta-rule recurrence with output norm and
gate) and the per-head q/k RMSNorm; CUDA kernels in csrc/gdn.cu, fp32 PyTorch restatements here as the oracle
(reference kernels: native/hip/src/linear_attention_kernel.hip.cpp:77,128; state contract
crates/sllm-core/src/linear_attention.rs)."""
from __future__ import annotations

import ctypes as C
import math

from typing import Optional

import torch

from . import _lib

P, I, F = C.c_void_p, C.c_int, C.c_float
_SIGS = {
    "sllm_gdn_conv_silu": (I, [P, P, P, P, P, P, I, I, I, I, P]),
    "sllm_gdn_recurrent": (I, [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P]),
    "sllm_gdn_recurrent_prompt": (I, [P] * 11 + [I] * 7 + [P, C.c_longlong, P]),
    "sllm_qk_headnorm": (I, [P, I, I, I, I, I, P, P, F, I, P]),
    "sllm_qkv_headnorm": (I, [P, I, I, I, I, I, P, P, F, I, I, I, P]),
}


def _k():
    for n, s in _SIGS.items():
        _lib.EXTRA_KERNEL_SIGNATURES.setdefault(n, s)
    return _lib.kernels()


def _bf(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


def conv_silu(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, row_off: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """x [T, width]; w [width, taps]; state [slots, taps - 1, width] updated in place; returns silu(conv) [T, width]."""
    t, width = x.shape
    taps = w.shape[1]
    if _lib.on_cpu(x):
        y = torch.empty((t, width), dtype=torch.float32)
        xf, wf = x.float(), w.float()
        offs = row_off.tolist()
        for s, slot in enumerate(slots.tolist()):
            r0, r1 = offs[s], offs[s + 1]
            seq = torch.cat([state[slot].float(), xf[r0:r1]], dim=0)
            for r in range(r1 - r0):
                acc = torch.zeros(width)
                for tap in range(taps):
                    acc = acc + seq[r + tap] * wf[:, tap]
                y[r0 + r] = acc / (1 + torch.exp(-acc))
            state[slot] = seq[-(taps - 1):].to(state.dtype)
        return y if x.dtype == torch.float32 else y.to(torch.bfloat16)
    from .core import _p, _stream
    if x.stride(1) != 1:
        x = x.contiguous()
    y = torch.empty((t, width), dtype=x.dtype, device=x.device)       # x may be a column slice of a wider matrix
    rc = _k().sllm_gdn_conv_silu(_p(x), _p(w), _p(state), _p(y), _p(row_off), _p(slots), slots.numel(), width, taps,
                                 x.stride(0), _stream())
    _lib.check(rc, "gdn_conv_silu")
    return y


PROMPT_FORM_MIN_ROWS_PER_SEQUENCE = 8
_prompt_form = {"on": True}


def prompt_form_enabled() -> bool:
    return _prompt_form["on"]


def set_prompt_form(on: bool) -> None:
    """Whether flat batches that average 8 or more rows per sequence take the three-stage form of the recurrence."""
    _prompt_form["on"] = bool(on)


def recurrent(qkv, z, b, a, a_log, dt_bias, norm_w, state, row_off, slots, qk_heads: int, v_heads: int, hd: int = 128):
    """Gated delta rule over a flat batch; state [slots, v_heads, hd, hd] fp32 updated in place; returns [T, v_heads*hd]."""
    t = qkv.shape[0]
    if _lib.on_cpu(qkv):
        out = torch.empty((t, v_heads * hd), dtype=torch.float32)
        rep = v_heads // qk_heads
        offs = row_off.tolist()
        q_all = qkv.float()[:, :qk_heads * hd].view(t, qk_heads, hd)
        k_all = qkv.float()[:, qk_heads * hd:2 * qk_heads * hd].view(t, qk_heads, hd)
        v_all = qkv.float()[:, 2 * qk_heads * hd:].view(t, v_heads, hd)
        zf = z.float().view(t, v_heads, hd)
        for s, slot in enumerate(slots.tolist()):
            for r in range(offs[s], offs[s + 1]):
                for vh in range(v_heads):
                    qh = vh // rep
                    q, k, v = q_all[r, qh], k_all[r, qh], v_all[r, vh]
                    qn = _bf(q / torch.sqrt((q * q).sum() + 1e-6)) / math.sqrt(hd)
                    kn = _bf(k / torch.sqrt((k * k).sum() + 1e-6))
                    beta = _bf(torch.sigmoid(b.float()[r, vh]))
                    av = a.float()[r, vh] + dt_bias.float()[vh]
                    decay = torch.exp(-torch.exp(a_log.float()[vh]) * torch.nn.functional.softplus(av))
                    S = state[slot, vh] * decay
                    resid = beta * (v - S @ kn)
                    S = S + resid[:, None] * kn[None, :]
                    state[slot, vh] = S
                    o = _bf(S @ qn)
                    inv = 1.0 / torch.sqrt((o * o).sum() / hd + 1e-6)
                    zz = zf[r, vh]
                    out[r, vh * hd:(vh + 1) * hd] = _bf(o * inv) * norm_w.float() * (zz / (1 + torch.exp(-zz)))
        return out if qkv.dtype == torch.float32 else out.to(torch.bfloat16)
    from .core import _p, _stream
    out = torch.empty((t, v_heads * hd), dtype=torch.bfloat16, device=qkv.device)
    # z, b and a may be column slices of the input projection's output: the kernels take their row strides
    if z.stride(1) != 1:
        z = z.contiguous()
    if b.stride(1) != 1 or a.stride(1) != 1 or a.stride(0) != b.stride(0):
        b, a = b.contiguous(), a.contiguous()
    qkv = qkv if qkv.is_contiguous() else qkv.contiguous()
    ldz, ldg = z.stride(0), b.stride(0)
    if t >= PROMPT_FORM_MIN_ROWS_PER_SEQUENCE * slots.numel() and prompt_form_enabled():
        # prompts: the state-independent work (q / k normalisation, gates, output norm) runs in parallel over the
        # tokens, the scan itself carries no reduction (three launches; a decode step keeps the fused kernel)
        n = t * (2 * qk_heads * hd + 2 * v_heads + v_heads * hd)
        scratch = torch.empty((n,), dtype=torch.float32, device=qkv.device)
        rc = _k().sllm_gdn_recurrent_prompt(_p(qkv), _p(z), _p(b), _p(a), _p(a_log), _p(dt_bias), _p(norm_w), _p(state), _p(out),
                                            _p(row_off), _p(slots), slots.numel(), t, qk_heads, v_heads, hd, ldz, ldg,
                                            _p(scratch), n, _stream())
        _lib.check(rc, "gdn_recurrent_prompt")
        return out
    rc = _k().sllm_gdn_recurrent(_p(qkv), _p(z), _p(b), _p(a), _p(a_log), _p(dt_bias), _p(norm_w), _p(state), _p(out),
                                 _p(row_off), _p(slots), slots.numel(), qk_heads, v_heads, hd, ldz, ldg, _stream())
    _lib.check(rc, "gdn_recurrent")
    return out


def qk_headnorm(qkv: torch.Tensor, hq: int, hkv: int, hd: int, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
                eps: float, offset_one: bool = False, norm_v: bool = False) -> torch.Tensor:
    """RMS-normalises every q and k head of a fused [T, (hq + 2 hkv) * hd] activation in place; returns it.
    A missing weight vector means "all ones" (with wq and wk both None the q / k heads are left alone);
    ``norm_v`` also normalises the value heads, without a weight (Gemma-4's v_norm)."""
    t = qkv.shape[0]
    if _lib.on_cpu(qkv):
        x = qkv.view(t, hq + 2 * hkv, hd)
        spans = [] if (wq is None and wk is None) else [(0, hq, wq), (hq, hq + hkv, wk)]
        if norm_v:
            spans.append((hq + hkv, hq + 2 * hkv, None))
        for lo, hi, w in spans:
            v = x[:, lo:hi].float()
            g = 1.0 if w is None else w.float() + (1.0 if offset_one else 0.0)
            x[:, lo:hi] = (v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * g).to(qkv.dtype)
        return qkv
    from .core import _p, _stream
    skip_qk = wq is None and wk is None
    rc = _k().sllm_qkv_headnorm(_p(qkv), qkv.stride(0), t, hq, hkv, hd, _p(wq), _p(wk), eps, int(offset_one),
                                int(skip_qk), int(norm_v), _stream())
    _lib.check(rc, "qkv_headnorm")
    return qkv

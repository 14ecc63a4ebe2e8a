"""Mixture-of-experts ops: routing, permutation, grouped expert GEMMs, combine - CUDA kernels with CPU oracles.

The CPU path is the oracle of the same contract (reference: reference_sparse_moe_route,
crates/sllm-core/src/moe.rs:229: top-k by logit, ties to the lower index, softmax over the selected logits).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from .w4 import W4Weight, linear_w4

P, I, L = C.c_void_p, C.c_int, C.c_longlong
_SIGS = {
    "sllm_moe_route": (I, [P, I, I, I, I, I, P, P, P]),
    "sllm_moe_permute": (I, [P, P, I, I, I, I, P, P, P, P, P]),
    "sllm_moe_gather": (I, [P, I, P, P, I, P, I, I, P]),
    "sllm_moe_combine": (I, [P, P, I, P, P, I, I, P]),
    "sllm_moe_shared_add": (I, [P, P, P, I, P, I, I, P]),
    "sllm_moe_owner_plan": (I, [P, P, P, I, I, L, L, P, I, I, I, I, P, P, P]),
    "sllm_moe_owner_combine": (I, [P, P, P, I, I, L, L, I, P, P, I, I, I, I, P, P, P, P]),
    "sllm_moe_combine_allreduce": (I, [P, P, I, I, P, P, I, P, P, I, I, I, L, I, P, P, P]),
}


def _k():
    for n, s in _SIGS.items():
        _lib.EXTRA_KERNEL_SIGNATURES.setdefault(n, s)
    return _lib.kernels()


def route(logits: torch.Tensor, top_k: int, softmax_all: bool = False):
    """[T, E] -> (idx int32 [T, k], weights fp32 [T, k])."""
    t, e = logits.shape
    if _lib.on_cpu(logits):
        lf = torch.nan_to_num(logits.float(), nan=float("-inf"))
        # stable ordering: larger logit first, ties to the lower index
        order = torch.sort(-lf, dim=1, stable=True).indices[:, :top_k]
        sel = torch.gather(lf, 1, order)
        if softmax_all:
            w = torch.softmax(lf, dim=1).gather(1, order)
        else:
            w = torch.softmax(sel, dim=1)
        return order.to(torch.int32), w.float()
    from .core import _p, _stream
    idx = torch.empty((t, top_k), dtype=torch.int32, device=logits.device)
    w = torch.empty((t, top_k), dtype=torch.float32, device=logits.device)
    rc = _k().sllm_moe_route(_p(logits), logits.stride(0), t, e, top_k, int(softmax_all), _p(idx), _p(w), _stream())
    _lib.check(rc, "moe_route")
    return idx, w


def permute(idx: torch.Tensor, w: torch.Tensor, e_lo: int, e_hi: int):
    """Groups assignments by local expert.  Returns (tok_off [n_local + 1], perm_src [T*k], perm_dst [T, k],
    perm_w [T*k]); rows beyond tok_off[-1] are unused."""
    t, k = idx.shape
    n_local = e_hi - e_lo
    dev = idx.device
    tok_off = torch.zeros(n_local + 1, dtype=torch.int32, device=dev)
    perm_src = torch.zeros(t * k, dtype=torch.int32, device=dev)
    perm_dst = torch.full((t, k), -1, dtype=torch.int32, device=dev)
    perm_w = torch.zeros(t * k, dtype=torch.float32, device=dev)
    if _lib.on_cpu(idx):
        flat = idx.reshape(-1).tolist()
        wf = w.reshape(-1).tolist()
        cur = 0
        for e in range(e_lo, e_hi):
            tok_off[e - e_lo] = cur
            for a, ex in enumerate(flat):
                if ex == e:
                    perm_src[cur] = a // k
                    perm_w[cur] = wf[a]
                    perm_dst[a // k, a % k] = cur
                    cur += 1
        tok_off[n_local] = cur
        return tok_off, perm_src, perm_dst, perm_w
    from .core import _p, _stream
    rc = _k().sllm_moe_permute(_p(idx), _p(w), t, k, e_lo, e_hi, _p(tok_off), _p(perm_src), _p(perm_dst), _p(perm_w), _stream())
    _lib.check(rc, "moe_permute")
    return tok_off, perm_src, perm_dst, perm_w


def gather(x: torch.Tensor, perm_src: torch.Tensor, tok_off: torch.Tensor) -> torch.Tensor:
    rows = perm_src.numel()
    if _lib.on_cpu(x):
        return x[perm_src.long()]
    from .core import _p, _stream
    xp = torch.empty((rows, x.shape[1]), dtype=torch.bfloat16, device=x.device)
    rc = _k().sllm_moe_gather(_p(x), x.stride(0), _p(perm_src), _p(tok_off), tok_off.numel() - 1, _p(xp), x.shape[1], rows,
                              _stream())
    _lib.check(rc, "moe_gather")
    return xp


def combine(yp: torch.Tensor, perm_dst: torch.Tensor, residual: Optional[torch.Tensor]) -> torch.Tensor:
    t, k = perm_dst.shape
    d = yp.shape[1]
    if _lib.on_cpu(yp):
        out = torch.zeros((t, d), dtype=torch.float32)
        for j in range(k):
            p = perm_dst[:, j].long()
            m = p >= 0
            out[m] += yp.float()[p[m]]
        if residual is not None:
            out = out + residual.float()
        return out if yp.dtype == torch.float32 else out.to(torch.bfloat16)
    from .core import _p, _stream
    y = torch.empty((t, d), dtype=torch.bfloat16, device=yp.device)
    rc = _k().sllm_moe_combine(_p(yp), _p(perm_dst), k, _p(residual), _p(y), t, d, _stream())
    _lib.check(rc, "moe_combine")
    return y


def shared_add(a: torch.Tensor, b: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """a + sigmoid(gate) * b with one gate logit per row: a, b [T, d]; gate [T] (any stride, e.g. a column of the
    router logits)."""
    if _lib.on_cpu(a):
        out = a.float() + torch.sigmoid(gate.float()).unsqueeze(1) * b.float()
        return out if a.dtype == torch.float32 else out.to(torch.bfloat16)
    from .core import _p, _stream
    y = torch.empty_like(a)
    rc = _k().sllm_moe_shared_add(_p(a), _p(b), _p(gate), gate.stride(0), _p(y), a.shape[0], a.shape[1], _stream())
    _lib.check(rc, "moe_shared_add")
    return y


def expert_mlp(x: torch.Tensor, tok_off: torch.Tensor, perm_src: torch.Tensor, perm_w: torch.Tensor, gate_up: W4Weight,
               down: W4Weight, act: str, row_ptr: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """The gated MLP of the local experts over the routed rows (grouped by expert: `tok_off`), routing weights applied:
    y_perm [T*k, d], or None when `row_ptr` scatters the rows (see `linear_w4`).

    W4A16 (default): gather rows -> grouped gate_up GEMM -> SiLU*up -> grouped down GEMM, bf16 activations.
    W4A4 (`ops.w4.set_w4a4`): the quantiser reads the routed rows in place (no gather), both GEMMs run on the
    block-scaled 4-bit tensor-core kernel, and SiLU*up is computed inside the quantiser of the down projection
    (reference: the fused expert kernels, native/hip/src/moe_expert_kernel.hip.cpp:88,176)."""
    from . import core
    from . import w4 as W
    t = x.shape[0]
    # 4-bit activations serve the decode regime; with more than 32 routed rows per expert on average (a prompt) the
    # rows are compute bound and keep bf16 activations on the W4A16 kernel, whose token tiles are 128 wide
    if W.w4a4_enabled() and x.dtype == torch.bfloat16 and perm_src.numel() <= W.W4A4_MAX_DENSE_ROWS * gate_up.groups:
        rows = perm_src.numel()
        n_rows = tok_off[-1:] if x.is_cuda else None
        if not x.is_cuda:
            rows = int(tok_off[-1])
        q = W.act_quant_fp4(x, gate_up.fmt, src_row=perm_src, tokens=rows, n_rows=n_rows)
        gu = W.linear_w4a4(None, gate_up, tok_off=tok_off, max_group_tokens=t, quantized=q)
        q2 = W.act_quant_fp4(gu, down.fmt, n_rows=n_rows, gated=act)
        y = W.linear_w4a4(None, down, tok_off=tok_off, tok_scale=perm_w[:rows], max_group_tokens=t, quantized=q2,
                          row_ptr=row_ptr)
        if y is not None and y.shape[0] < perm_src.numel():
            y = torch.cat([y, y.new_zeros((perm_src.numel() - y.shape[0], y.shape[1]))])
        return y
    xp = gather(x, perm_src, tok_off)
    a = core.gated_act(linear_w4(xp, gate_up, tok_off=tok_off, max_group_tokens=t), act)
    return linear_w4(a, down, tok_off=tok_off, tok_scale=perm_w, max_group_tokens=t, row_ptr=row_ptr)


def experts_forward(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, gate_up: W4Weight, down: W4Weight, act: str,
                    e_lo: int, e_hi: int):
    """Runs the local experts [e_lo, e_hi) on the tokens routed to them.  Returns (y_perm [T*k, d] with the routing
    weights applied, perm_dst [T, k])."""
    tok_off, perm_src, perm_dst, perm_w = permute(idx, w, e_lo, e_hi)
    return expert_mlp(x, tok_off, perm_src, perm_w, gate_up, down, act), perm_dst

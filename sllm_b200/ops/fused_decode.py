"""Front end of the fused decode kernel (csrc/decode_fused.cu): descriptor structs, a launch call, and the
CPU restatement of every phase used by the tests.

One launch chains up to four block-scaled FP8 GEMMs of a decoder layer inside one persistent kernel; the
epilogue of each phase writes the operand of the next one (see csrc/decode_fused.h for the phase kinds).
The reference runs the same ops as one kernel each (crates/sllm-core/src/qwen_graph.rs:2524-3501).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib, reference as ref
from .core import _p, _stream, workspace

PLAIN, RESID_QUANT, SILU_QUANT, ROPE_KV = 0, 1, 2, 3
MAX_PHASES = 4
MAX_ROWS = 32


class FdPhase(C.Structure):
    _fields_ = [("epilogue", C.c_int), ("n", C.c_int), ("k", C.c_int), ("dual_off", C.c_int),
                ("norm_tiles", C.c_int), ("norm_dim", C.c_int), ("act", C.c_int), ("ldy", C.c_int),
                ("eps", C.c_float), ("softcap", C.c_float),
                ("ld_sa", C.c_int), ("ld_sb", C.c_int), ("ld_s_out", C.c_int), ("reserved", C.c_int),
                ("w", C.c_void_p), ("w_scale", C.c_void_p), ("x", C.c_void_p), ("x_scale", C.c_void_p),
                ("ssq_in", C.c_void_p), ("y", C.c_void_p), ("residual", C.c_void_p), ("q_out", C.c_void_p),
                ("s_out", C.c_void_p), ("ssq_out", C.c_void_p)]


class FdRope(C.Structure):
    _fields_ = [("positions", C.c_void_p), ("seq_index", C.c_void_p), ("block_table", C.c_void_p),
                ("max_blocks", C.c_int), ("hq", C.c_int), ("hkv", C.c_int), ("rotary_dim", C.c_int),
                ("page_size", C.c_int), ("kv_fp8", C.c_int),
                ("theta", C.c_float), ("k_static", C.c_float), ("v_static", C.c_float), ("reserved", C.c_int),
                ("k_pages", C.c_void_p), ("v_pages", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
                ("inv_freq", C.c_void_p)]


class FdDesc(C.Structure):
    _fields_ = [("n_phases", C.c_int), ("rows", C.c_int), ("n_counters", C.c_int), ("grid", C.c_int),
                ("phase", FdPhase * MAX_PHASES), ("rope", FdRope),
                ("ws", C.c_void_p), ("ws_floats", C.c_longlong), ("counters", C.c_void_p),
                ("sync", C.c_void_p), ("status", C.c_void_p), ("comm", C.c_void_p),
                ("wait_limit_cycles", C.c_longlong)]


_lib.EXTRA_KERNEL_SIGNATURES.update({
    "sllm_fused_decode": (C.c_int, [C.POINTER(FdDesc), C.c_void_p]),
    "sllm_fused_decode_ws_floats": (C.c_longlong, [C.c_int]),
    "sllm_embed_quant": (C.c_int, [C.c_void_p] * 6 + [C.c_int] * 4 + [C.c_float, C.c_void_p]),
    "sllm_fused_decode_abi": (C.c_int, [C.POINTER(C.c_int), C.c_int]),
    "sllm_fused_decode_set_trace": (None, [C.c_void_p]),
    "sllm_fused_decode_set_lookahead": (None, [C.c_int]),
    "sllm_gemm_fused": (C.c_int, [C.POINTER(FdPhase), C.POINTER(FdRope), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                  C.c_longlong, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
})

_abi_checked = False


def _comm_layout():
    from ..parallel.tp import CommDesc
    return [C.sizeof(CommDesc), CommDesc.recv.offset, CommDesc.epoch.offset]


def check_abi() -> None:
    """Compares the ctypes mirrors with the sizes and offsets the library was compiled with; a mismatch would hand
    pointers to the wrong fields."""
    global _abi_checked
    if _abi_checked:
        return
    lib = _lib.kernels()
    buf = (C.c_int * 32)()
    n = lib.sllm_fused_decode_abi(buf, 32)
    mine = [C.sizeof(FdPhase), FdPhase.eps.offset, FdPhase.w.offset, FdPhase.ssq_out.offset,
            C.sizeof(FdRope), FdRope.theta.offset, FdRope.k_pages.offset, FdRope.inv_freq.offset,
            C.sizeof(FdDesc), FdDesc.phase.offset, FdDesc.rope.offset, FdDesc.ws.offset, FdDesc.sync.offset,
            FdDesc.comm.offset, FdDesc.wait_limit_cycles.offset] + _comm_layout()
    theirs = list(buf[:n])
    if n != len(mine) or theirs != mine:
        raise _lib.KernelError(f"fused-decode descriptor layout mismatch: library {theirs}, bindings {mine}")
    _abi_checked = True


@dataclass
class FdState:
    """Per-device scratch of the fused decode kernel: stream-K partials, tile counters, the grid-barrier word."""
    ws: torch.Tensor
    counters: torch.Tensor
    sync: torch.Tensor


_states: dict = {}


def state(device: torch.device) -> FdState:
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _states.get(key)
    if st is None:
        lib = _lib.kernels()
        floats = int(lib.sllm_fused_decode_ws_floats(0))
        st = FdState(torch.zeros(floats, dtype=torch.float32, device=device),
                     torch.zeros(4096, dtype=torch.int32, device=device),
                     torch.zeros(2, dtype=torch.int64, device=device))
        _states[key] = st
    return st


def reset_state(device: torch.device) -> None:
    """After a launch whose bounded wait gave up, the counters and the barrier word are undefined: zero them."""
    st = state(device)
    st.counters.zero_()
    st.sync.zero_()


def _ld(t: torch.Tensor) -> int:
    """Leading dimension of a 2-D plane; a single-row tensor may report any stride for dimension 0."""
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def set_trace(buf: Optional[torch.Tensor]) -> None:
    """Profiling aid: later launches write per-CTA, per-phase globaltimer stamps into ``buf`` (int64 [CTAs, 4, 8]);
    None switches it off."""
    _lib.kernels().sllm_fused_decode_set_trace(None if buf is None else buf.data_ptr())


def set_lookahead(tiles: int) -> None:
    """Tuning knob: how many 16 KB weight tiles per CTA the producer prefetches into L2 ahead of its ring."""
    _lib.kernels().sllm_fused_decode_set_lookahead(int(tiles))


def phase(epilogue: int, w, w_scale, x, x_scale, *, n: int, k: int, dual_off: int = 0, ssq_in=None, norm_dim: int = 0,
          eps: float = 1e-5, act: int = 0, y=None, ldy: int = 0, residual=None, q_out=None, s_out=None, ssq_out=None,
          ld_s_out: int = 0, softcap: float = 0.0) -> FdPhase:
    ph = FdPhase()
    ph.epilogue, ph.n, ph.k, ph.dual_off = epilogue, n, k, dual_off
    ph.norm_tiles = (norm_dim + 127) // 128 if ssq_in is not None else 0
    ph.norm_dim, ph.act, ph.ldy, ph.eps, ph.softcap = norm_dim, act, ldy, eps, softcap
    ph.ld_sa, ph.ld_sb = _ld(w_scale), _ld(x_scale)
    ph.ld_s_out = ld_s_out if ld_s_out else ph.ld_sb
    for name, t in (("w", w), ("w_scale", w_scale), ("x", x), ("x_scale", x_scale), ("ssq_in", ssq_in), ("y", y),
                    ("residual", residual), ("q_out", q_out), ("s_out", s_out), ("ssq_out", ssq_out)):
        setattr(ph, name, None if t is None else t.data_ptr())
    return ph


_inv_freq_cache: dict = {}


def inv_freq_table(theta: float, rotary_dim: int, device) -> torch.Tensor:
    """theta^(-2 i / rotary_dim), i < rotary_dim / 2, evaluated in float64 and rounded once to fp32."""
    key = (float(theta), int(rotary_dim), str(device))
    t = _inv_freq_cache.get(key)
    if t is None:
        i = torch.arange(rotary_dim // 2, dtype=torch.float64)
        t = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / rotary_dim).to(torch.float32).to(device)
        if t.is_cuda:
            # the kernels stage this table in their preamble, which may run before the work queued ahead of them has
            # finished: the upload must have landed before the first launch that names it
            torch.cuda.current_stream(t.device).synchronize()
        _inv_freq_cache[key] = t
    return t


def rope_desc(positions, seq_index, block_table, kv, hq: int, hkv: int, rotary_dim: int, theta: float,
              inv_freq=None) -> FdRope:
    r = FdRope()
    if inv_freq is None:
        inv_freq = inv_freq_table(theta, rotary_dim, positions.device)
    r.positions, r.seq_index, r.block_table = positions.data_ptr(), seq_index.data_ptr(), block_table.data_ptr()
    r.max_blocks, r.hq, r.hkv, r.rotary_dim = block_table.stride(0), hq, hkv, rotary_dim
    r.page_size, r.kv_fp8, r.theta = kv.page_size, int(kv.fp8), theta
    r.k_static, r.v_static = kv.k_static, kv.v_static
    r.k_pages, r.v_pages = kv.k.data_ptr(), kv.v.data_ptr()
    r.k_scale = None if kv.k_scale is None else kv.k_scale.data_ptr()
    r.v_scale = None if kv.v_scale is None else kv.v_scale.data_ptr()
    r.inv_freq = inv_freq.data_ptr()
    return r


_il_cache: dict = {}


def interleave_gate_up(w: torch.Tensor, scale_t: torch.Tensor, ffn: int):
    """Row order of the gate / up matrix for the cluster-GEMM SiLU epilogue: per 128-row tile, the 64 gate rows of 64
    features followed by the 64 up rows of the same features.  Returns (weight, scales) in that order."""
    if ffn % 128:
        raise ValueError("the gated width must be a multiple of 128")
    j = torch.arange(ffn // 64, device=w.device).repeat_interleave(64) * 64 + torch.arange(64, device=w.device).repeat(ffn // 64)
    idx = torch.stack([j.view(-1, 64), (j + ffn).view(-1, 64)], dim=1).reshape(-1)
    return w[idx].contiguous(), scale_t[:, idx].contiguous()


def backend() -> str:
    """'cluster': one cluster split-K GEMM launch per phase (gemm_tcgen05.cu); 'persistent': all phases of a launch in
    one persistent kernel (decode_fused.cu).  Chosen by SLLM_FD_BACKEND (default cluster)."""
    import os
    return os.environ.get("SLLM_FD_BACKEND", "cluster")


def _resolve_cluster_phase(ph: FdPhase, i: int, rows: int, il: Optional[list]):
    """(descriptor with the weight the cluster GEMM reads, weight rows, bn, splits, stages) of a phase."""
    from .core import _gemm_plan
    one = FdPhase.from_buffer_copy(ph)
    w_rows = ph.n
    if ph.epilogue == SILU_QUANT:
        pair = il[i] if il is not None and il[i] is not None else None
        if pair is None:
            key = (ph.w, ph.w_scale, ph.n)
            pair = _il_cache.get(key)
            if pair is None:
                raise ValueError("the cluster backend needs the interleaved gate / up weight (interleave_gate_up)")
        one.w, one.w_scale = pair[0].data_ptr(), pair[1].data_ptr()
        one.ld_sa = _ld(pair[1])
        w_rows = 2 * ph.n
    _, bn, splits, stages = _gemm_plan(rows, w_rows, ph.k // 128)
    if ph.epilogue == SILU_QUANT:
        splits = 1
    return one, w_rows, bn, splits, stages


def _launch_cluster(phases: list, rows: int, device: torch.device, rope: Optional[FdRope], il: Optional[list],
                    comm=None) -> None:
    wsp = workspace(device)
    lib = _lib.kernels()
    plans = [_resolve_cluster_phase(ph, i, rows, il) for i, ph in enumerate(phases)]
    for one, w_rows, bn, splits, stages in plans:
        if _lib.audit_enabled():
            _lib.record_dispatch("fused_decode_phase", "gemm_tcgen05_kernel", epilogue=int(one.epilogue), rows=rows, n=w_rows,
                                 k=int(one.k), bn=bn, splits=splits, stages=stages, tensor_parallel=comm is not None,
                                 grid=[(w_rows + 127) // 128, 1, splits])
        rc = lib.sllm_gemm_fused(C.byref(one), C.byref(rope) if rope is not None else None, rows, bn, splits, stages,
                                 _p(wsp.ws), wsp.ws.numel(), _p(wsp.counters), wsp.counters.numel(), _p(wsp.status),
                                 _stream(), None if comm is None else C.cast(C.pointer(comm), C.c_void_p))
        _lib.check(rc, "gemm_fused")


def launch(phases: list, rows: int, device: torch.device, rope: Optional[FdRope] = None, comm=None, grid: int = 0,
           wait_limit_cycles: int = 0, impl: Optional[str] = None, interleaved: Optional[list] = None) -> None:
    """Runs the phases (1..4) on the current stream: as one persistent kernel, or as one cluster GEMM per phase
    (``impl`` / SLLM_FD_BACKEND).  ``interleaved[i]``: (weight, scales) of a SILU_QUANT phase in the row order of
    ``interleave_gate_up`` (cluster backend)."""
    check_abi()
    if not 1 <= len(phases) <= MAX_PHASES or not 1 <= rows <= MAX_ROWS:
        raise ValueError("a fused decode launch takes 1..4 phases and 1..32 rows")
    impl = impl or backend()
    if impl == "cluster":
        return _launch_cluster(phases, rows, device, rope, interleaved, comm)
    st = state(device)
    d = FdDesc()
    d.n_phases, d.rows, d.n_counters, d.grid = len(phases), rows, st.counters.numel(), grid
    for i, ph in enumerate(phases):
        d.phase[i] = ph
    if rope is not None:
        d.rope = rope
    d.ws, d.ws_floats, d.counters = st.ws.data_ptr(), st.ws.numel(), st.counters.data_ptr()
    d.sync, d.status = st.sync.data_ptr(), workspace(device).status.data_ptr()
    d.comm = None if comm is None else C.cast(C.pointer(comm), C.c_void_p)
    d.wait_limit_cycles = wait_limit_cycles
    rc = _lib.kernels().sllm_fused_decode(C.byref(d), _stream())
    _lib.check(rc, "fused_decode")


def embed_quant(table: torch.Tensor, ids: torch.Tensor, h, q_out, s_out, ssq_out, scale: float = 1.0) -> None:
    rows, d = ids.numel(), table.shape[1]
    rc = _lib.kernels().sllm_embed_quant(_p(table), _p(ids), _p(h), _p(q_out), _p(s_out), _p(ssq_out), _ld(s_out),
                                         rows, d, table.shape[0], scale, _stream())
    _lib.check(rc, "embed_quant")


# ------------------------------------------------------------------------------------------------
# fp32 restatements of the phases (oracle for the tests)
# ------------------------------------------------------------------------------------------------
def _deq_w(w: torch.Tensor, w_scale_t: torch.Tensor) -> torch.Tensor:
    return ref.dequant_fp8_1x128(w.cpu(), w_scale_t.cpu()[:, :w.shape[0]].contiguous())


def _deq_x(x: torch.Tensor, x_scale_t: torch.Tensor, rows: int) -> torch.Tensor:
    return ref.dequant_fp8_1x128(x.cpu()[:rows], x_scale_t.cpu()[:, :rows].contiguous())


def ref_norm_factor(ssq: torch.Tensor, rows: int, dim: int, eps: float) -> torch.Tensor:
    return torch.rsqrt(ssq.cpu()[:(dim + 127) // 128, :rows].sum(dim=0) / dim + eps)


def ref_plain(w, ws, x, xs, rows, *, norm=None, residual=None, softcap=0.0):
    y = _deq_x(x, xs, rows) @ _deq_w(w, ws).t()
    if norm is not None:
        y = y * norm.unsqueeze(1)
    if residual is not None:
        y = y + residual.cpu()[:rows].to(torch.float32)
    if softcap > 0:
        y = softcap * torch.tanh(y / softcap)
    return y


def ref_quant_rows(v: torch.Tensor):
    """bf16-rounded values -> (E4M3 bytes, scales [n/128, rows], sums of squares [n/128, rows])."""
    v = ref.round_bf16(v)
    q, s_t = ref.quant_fp8_1x128(v)
    ssq = v.view(v.shape[0], -1, 128).pow(2).sum(dim=-1).t().contiguous()
    return v, q, s_t, ssq


def ref_silu(w, ws, x, xs, rows, n, dual_off, norm, act: int = 0):
    full = _deq_x(x, xs, rows) @ _deq_w(w, ws).t()
    g, u = full[:, :n], full[:, dual_off:dual_off + n]
    if norm is not None:
        g, u = g * norm.unsqueeze(1), u * norm.unsqueeze(1)
    a = ref.silu(g) if act == 0 else ref.gelu_tanh(g)
    return ref.round_bf16(a) * u

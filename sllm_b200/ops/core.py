"""Device-dispatching op layer used by the model graphs.

CUDA tensors always run the hand-written sm_100a kernels through the C ABI (and fail loudly when
the library is missing); CPU tensors run the PyTorch restatements in ``reference.py``.  The split is
by device, not by a backend registry: there is one GPU target.

Semantic-op coverage relative to the reference's op list (crates/sllm-core/src/op.rs:6-24): Copy, Add,
ScalarMul, Embedding, Matmul, SiluMul, GeluTanhMul, SigmoidMul, TanhSoftcap, RmsNorm, Rotary,
CausalAttention, AttentionPreprocess (rope_kv_append), Argmax, TokenSelect (ops.sampling), SparseMoe
(ops.moe), BroadcastAdd.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import NamedTuple, Optional

import torch

from . import _lib, reference as ref


class QTensor(NamedTuple):
    """Block-scaled FP8 activation: E4M3 bytes [M, K] + fp32 scales [ceil(K/128), M]."""
    data: torch.Tensor
    scale: torch.Tensor


@dataclass
class LinearWeight:
    """A [N, K] weight in one of the resident encodings.

    kind 'dense': bf16 (GPU) or fp32 (CPU oracle) values in ``w``.
    kind 'fp8'  : E4M3FN bytes in ``w`` + ``scale_t`` = fp32 [ceil(K/128), N] (the file format's
                  [N, ceil(K/128)] 1x128 scales, transposed once at load so that one K block's scales
                  are contiguous for the GEMM epilogue).
    """
    kind: str
    w: Optional[torch.Tensor]
    scale_t: Optional[torch.Tensor] = None
    w4: object = None            # ops.w4.W4Weight for kind 'w4' (MXFP4 / NVFP4 codes, W4A16 GEMM)

    @property
    def out_features(self) -> int:
        return self.w4.n if self.kind == "w4" else self.w.shape[0]

    @property
    def in_features(self) -> int:
        return self.w4.k if self.kind == "w4" else self.w.shape[1]

    def dequantized(self) -> torch.Tensor:
        if self.kind == "w4":
            return self.w4.dequantized(0)
        if self.kind == "fp8":
            return ref.dequant_fp8_1x128(self.w, self.scale_t)
        return self.w.to(torch.float32)

    @staticmethod
    def from_dense(w: torch.Tensor, kind: str) -> "LinearWeight":
        if kind == "fp8":
            q, s_t = ref.quant_fp8_1x128(w)
            return LinearWeight("fp8", q, s_t)
        return LinearWeight("dense", w)

    def to(self, device) -> "LinearWeight":
        if self.kind == "w4":
            import dataclasses
            w4 = dataclasses.replace(self.w4, tiles=self.w4.tiles.to(device),
                                     tensor_scale=None if self.w4.tensor_scale is None else self.w4.tensor_scale.to(device))
            return LinearWeight("w4", None, None, w4)
        return LinearWeight(self.kind, self.w.to(device), None if self.scale_t is None else self.scale_t.to(device))


# ------------------------------------------------------------------------------------------------
# workspace (per device): split-K / split-KV partials, tile counters, device status word
# ------------------------------------------------------------------------------------------------
class Workspace:
    def __init__(self, device: torch.device, floats: int = 48 << 20, counters: int = 1 << 17):
        self.device = device
        self.ws = torch.empty(floats, dtype=torch.float32, device=device)
        self.counters = torch.zeros(counters, dtype=torch.int32, device=device)
        # word 0: first bounded-wait status; words 1..7: detail recorded with it (kernel specific)
        self.status = torch.zeros(8, dtype=torch.int32, device=device)


_workspaces: dict = {}


def workspace(device: torch.device) -> Workspace:
    if device.type != "cuda":            # only reached under a fake kernel library: a small host stand-in
        w = _workspaces.get(("cpu", 0))
        if w is None:
            w = _workspaces[("cpu", 0)] = Workspace(device, floats=1 << 16, counters=1 << 10)
        return w
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    w = _workspaces.get(key)
    if w is None:
        w = Workspace(torch.device("cuda", key[1]))
        _workspaces[key] = w
    return w


def device_status(device: torch.device) -> int:
    """Reads (and clears) the status word that bounded waits set when they give up.  Synchronises."""
    w = workspace(device)
    v = int(w.status[0].item())
    if v:
        w.status.zero_()
    return v


def _p(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream() -> C.c_void_p:
    if _lib.fake_active():
        return C.c_void_p(0)
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


_SM_COUNT = 148


# ------------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------------
def _gemm_plan(m: int, n: int, k_blocks: int):
    """(swap_ab, bn, splits, stages) for Y[m, n].  Stage counts keep a CTA near 105 KB of shared memory so that two
    CTAs share an SM (deeper pipelines that fill the SM with one CTA measured a third slower on the decode shapes)."""
    if m <= 128:
        bn = 16 if m <= 16 else 32 if m <= 32 else 64 if m <= 64 else 128
        tiles = (n + 127) // 128
        want = max(1, min((2 * _SM_COUNT) // max(tiles, 1), k_blocks // 4, 8))
        splits = 8 if want >= 8 else 4 if want >= 4 else 2 if want >= 2 else 1   # cluster sizes
        stages = {16: 5, 32: 4, 64: 3, 128: 5}[bn]
        return True, bn, splits, stages
    return False, 128, 1, 5


def gemm_raw(a: torch.Tensor, b: torch.Tensor, y: torch.Tensor, *, scale_a=None, scale_b=None, residual=None,
             transpose_out: bool, bn: int, splits: int, stages: int) -> None:
    """Direct access to the tcgen05 kernel: D[a_row, b_row] = sum_k A[a_row, k] B[b_row, k]."""
    lib = _lib.kernels()
    scaled = scale_a is not None
    a_rows, k = a.shape
    b_rows = b.shape[0]
    from ..core.types import reject_aliasing
    reject_aliasing(y, {"a": a, "b": b, "scale_a": scale_a, "scale_b": scale_b, "residual": residual}, may_equal=("residual",))
    wsp = workspace(a.device)
    rc = lib.sllm_gemm(_p(a), _p(b), _p(y), _p(scale_a), _p(scale_b), _p(residual), a_rows, b_rows, k,
                       1 if scaled else 0, 1 if transpose_out else 0, y.stride(0),
                       scale_a.stride(0) if scaled else 0, scale_b.stride(0) if scaled else 0, bn, splits, stages,
                       _p(wsp.ws), wsp.ws.numel(), _p(wsp.counters), wsp.counters.numel(), _p(wsp.status), _stream())
    _lib.check(rc, "gemm")


def linear(x, w: LinearWeight, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Y = X W^T (+ residual).  x: Tensor [M, K] (bf16 / fp32) or QTensor for FP8 weights."""
    xd = x.data if isinstance(x, QTensor) else x
    if w.kind == "w4":
        from .w4 import linear_w4
        return linear_w4(xd, w.w4, residual=residual)       # xd: a matrix, or activations quantised to 4 bits (Fp4Act)
    if _lib.on_cpu(xd):
        if isinstance(x, QTensor):
            xf = ref.dequant_fp8_1x128(x.data, x.scale)
        else:
            xf = x.to(torch.float32)
        if w.kind == "fp8" and not isinstance(x, QTensor):
            xf = ref.dequant_fp8_1x128(*ref.quant_fp8_1x128(x))
        y = xf @ w.dequantized().t()
        if residual is not None:
            y = y + residual.to(torch.float32)
        return y.to(residual.dtype if residual is not None else (torch.float32 if w.w.dtype == torch.float32 else torch.bfloat16))
    m = xd.shape[0]
    n = w.out_features
    if w.kind == "fp8":
        if not isinstance(x, QTensor):
            x = quant_fp8(x)
        k_blocks = (w.in_features + 127) // 128
    else:
        k_blocks = (w.in_features + 63) // 64
    y = torch.empty((m, n), dtype=torch.bfloat16, device=xd.device)
    swap, bn, splits, stages = _gemm_plan(m, n, k_blocks)
    if _lib.audit_enabled():
        _lib.record_dispatch("linear", "gemm_tcgen05_kernel", m=m, n=n, k=w.in_features, kind=w.kind, swap_ab=swap, bn=bn,
                             splits=splits, stages=stages, grid=[(n + 127) // 128 if swap else (m + 127) // 128,
                                                                 (m + bn - 1) // bn if swap else (n + bn - 1) // bn, splits])
    if w.kind == "fp8":
        if swap:
            gemm_raw(w.w, x.data, y, scale_a=w.scale_t, scale_b=x.scale, residual=residual, transpose_out=True,
                     bn=bn, splits=splits, stages=stages)
        else:
            gemm_raw(x.data, w.w, y, scale_a=x.scale, scale_b=w.scale_t, residual=residual, transpose_out=False,
                     bn=bn, splits=splits, stages=stages)
    else:
        if swap:
            gemm_raw(w.w, x, y, residual=residual, transpose_out=True, bn=bn, splits=splits, stages=stages)
        else:
            gemm_raw(x, w.w, y, residual=residual, transpose_out=False, bn=bn, splits=splits, stages=stages)
    return y


# ------------------------------------------------------------------------------------------------
# quantisation / norm / activation
# ------------------------------------------------------------------------------------------------
def _alloc_q(m: int, k: int, device) -> QTensor:
    return QTensor(torch.empty((m, k), dtype=torch.uint8, device=device),
                   torch.empty(((k + 127) // 128, m), dtype=torch.float32, device=device))


def quant_fp8(x: torch.Tensor) -> QTensor:
    if _lib.on_cpu(x):
        return QTensor(*ref.quant_fp8_1x128(x))
    m, k = x.shape
    q = _alloc_q(m, k, x.device)
    rc = _lib.kernels().sllm_quant_fp8_1x128(_p(x), _p(q.data), _p(q.scale), m, m, k, _stream())
    _lib.check(rc, "quant_fp8_1x128")
    return q


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, offset_one: bool = False, quant: bool = False):
    """RMSNorm over the last dim of [M, d]; quant=True returns a QTensor for a following FP8 GEMM."""
    if _lib.on_cpu(x):
        y = ref.rmsnorm(x, w, eps, offset_one)
        if x.dtype == torch.float32 and not quant:
            return y
        y = ref.round_bf16(y)
        return QTensor(*ref.quant_fp8_1x128(y)) if quant else y.to(x.dtype)
    m, d = x.shape
    lib = _lib.kernels()
    if quant:
        q = _alloc_q(m, d, x.device)
        rc = lib.sllm_rmsnorm(_p(x), _p(w), None, _p(q.data), _p(q.scale), m, m, d, eps, int(offset_one), _stream())
        _lib.check(rc, "rmsnorm")
        return q
    y = torch.empty_like(x)
    rc = lib.sllm_rmsnorm(_p(x), _p(w), _p(y), None, None, 0, m, d, eps, int(offset_one), _stream())
    _lib.check(rc, "rmsnorm")
    return y


def gated_act(x: torch.Tensor, act: str = "silu", quant: bool = False):
    """[M, 2I] (gate | up) -> act(gate) * up, optionally FP8-quantised for the down projection."""
    if _lib.on_cpu(x):
        y = ref.gated_act(x, act, round_intermediate=x.dtype != torch.float32)
        if x.dtype == torch.float32 and not quant:
            return y
        y = ref.round_bf16(y)
        return QTensor(*ref.quant_fp8_1x128(y)) if quant else y.to(x.dtype)
    m, two_i = x.shape
    inter = two_i // 2
    lib = _lib.kernels()
    a = 0 if act == "silu" else 1
    if quant:
        q = _alloc_q(m, inter, x.device)
        rc = lib.sllm_gated_act(_p(x), None, _p(q.data), _p(q.scale), m, m, inter, a, _stream())
        _lib.check(rc, "gated_act")
        return q
    y = torch.empty((m, inter), dtype=x.dtype, device=x.device)
    rc = lib.sllm_gated_act(_p(x), _p(y), None, None, 0, m, inter, a, _stream())
    _lib.check(rc, "gated_act")
    return y


def embedding(table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    if _lib.on_cpu(table):
        y = table[ids.long()]
        return y * scale if scale != 1.0 else y
    t = ids.numel()
    out = torch.empty((t, table.shape[1]), dtype=table.dtype, device=table.device)
    rc = _lib.kernels().sllm_embedding(_p(table), _p(ids), _p(out), t, table.shape[1], table.shape[0], scale, _stream())
    _lib.check(rc, "embedding")
    return out


_EW_OPS = {"add": 0, "scalar_mul": 1, "sigmoid_mul": 2, "tanh_softcap": 3, "broadcast_add": 4, "copy": 5}


def elementwise(op: str, a: torch.Tensor, b: Optional[torch.Tensor] = None, s: float = 0.0) -> torch.Tensor:
    if _lib.on_cpu(a):
        af = a.to(torch.float32)
        if op == "add" or op == "broadcast_add":
            r = af + b.to(torch.float32)
        elif op == "scalar_mul":
            r = af * s
        elif op == "sigmoid_mul":
            g = torch.sigmoid(b.to(torch.float32))
            r = af * (ref.round_bf16(g) if a.dtype != torch.float32 else g)
        elif op == "tanh_softcap":
            r = s * torch.tanh(af / s)
        else:
            r = af
        return r.to(a.dtype)
    y = torch.empty_like(a)
    rc = _lib.kernels().sllm_elementwise(_p(a), _p(b), _p(y), a.numel(), a.shape[-1], _EW_OPS[op], s, _stream())
    _lib.check(rc, "elementwise")
    return y


def argmax(logits: torch.Tensor, index_offset: int = 0, with_values: bool = False):
    """Row argmax: NaN in a row -> -1, ties -> lowest index."""
    if _lib.on_cpu(logits):
        lf = logits.to(torch.float32)
        idx = lf.argmax(dim=-1).to(torch.int32)
        # torch.argmax returns the first maximal index on CPU, matching the tie rule
        nan = torch.isnan(lf).any(dim=-1)
        idx = torch.where(nan, torch.full_like(idx, -1), idx + index_offset)
        return (idx, lf.max(dim=-1).values) if with_values else idx
    rows, n = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    val = torch.empty(rows, dtype=torch.float32, device=logits.device) if with_values else None
    wsp = workspace(logits.device)
    rc = _lib.kernels().sllm_argmax(_p(logits), _p(out), _p(val), rows, n, logits.stride(0), index_offset,
                                    _p(wsp.ws), wsp.ws.numel() * 4, _p(wsp.counters), wsp.counters.numel(), _stream())
    _lib.check(rc, "argmax")
    return (out, val) if with_values else out


# ------------------------------------------------------------------------------------------------
# RoPE + KV append, paged attention
# ------------------------------------------------------------------------------------------------
@dataclass
class KVLayer:
    """One layer's K/V pages.  values: [num_pages, hkv, page, hd] (uint8 E4M3 or bf16/fp32);
    scales: [num_pages, hkv, page] fp32 for dynamic FP8, None otherwise.  Head-major pages keep the
    page_size x head_dim bytes one attention CTA streams contiguous in HBM (2 KB for FP8, page 16)."""
    k: torch.Tensor
    v: torch.Tensor
    k_scale: Optional[torch.Tensor]
    v_scale: Optional[torch.Tensor]
    fp8: bool
    page_size: int
    k_static: float = 0.0
    v_static: float = 0.0
    # NVFP4 rows: values are uint8 [num_pages, hkv, page, hd / 2 + hd / 16] (E2M1 codes, element 2 i in the low nibble
    # of byte i, then one E4M3 scale per 16 channels); k_scale / v_scale hold the fp32 outer scale of every row
    # (reference: kv_state_kernel.hip.cpp:240-335, KvCacheEncoding::Nvfp4 of crates/sllm-core/src/kv_state.rs)
    nvfp4: bool = False

    @property
    def mode(self) -> int:
        """Page format code of the kernels: 0 bf16, 1 E4M3, 2 NVFP4."""
        return 2 if self.nvfp4 else int(self.fp8)


def rope_kv_append(qkv: torch.Tensor, positions: torch.Tensor, seq_index: torch.Tensor, block_table: torch.Tensor,
                   kv: KVLayer, hq: int, hkv: int, hd: int, theta: float, rotary_dim: Optional[int] = None,
                   inv_freq: Optional[torch.Tensor] = None, rope_pos3: Optional[torch.Tensor] = None,
                   mrope_sections: Optional[tuple] = None, pair_offset: int = 0) -> torch.Tensor:
    """Rotates q and k in ``qkv`` [T, (hq + 2 hkv) hd], appends k / v to the pages; returns q [T, hq*hd]
    (a view of qkv, rotated in place on CUDA).  ``rope_pos3`` (int32 [3, T]) with ``mrope_sections`` (temporal and
    height pair counts) gives 3-axis rotary positions; the page slot still follows ``positions``."""
    rd = rotary_dim or hd
    t = qkv.shape[0]
    if rope_pos3 is not None:
        if mrope_sections is None or tuple(rope_pos3.shape) != (3, t):
            raise ValueError("rope_pos3 must be [3, tokens] and needs mrope_sections")
        rope_pos3 = rope_pos3.contiguous()
    if _lib.on_cpu(qkv):
        x = qkv.view(t, hq + 2 * hkv, hd)
        q = ref.rope_split_half(x[:, :hq], positions, theta, rd, inv_freq, rope_pos3, mrope_sections, pair_offset)
        k = ref.rope_split_half(x[:, hq:hq + hkv], positions, theta, rd, inv_freq, rope_pos3, mrope_sections, pair_offset)
        v = x[:, hq + hkv:].to(torch.float32)
        if qkv.dtype != torch.float32:
            q, k = ref.round_bf16(q), ref.round_bf16(k)
        pos = positions.long()
        blk = block_table[seq_index.long(), pos // kv.page_size].long()
        off = pos % kv.page_size
        if kv.nvfp4:
            for plane, scale, x in ((kv.k, kv.k_scale, k), (kv.v, kv.v_scale, v)):
                rows, outer = ref.quant_kv_nvfp4_rows(x)
                plane[blk, :, off] = rows
                scale[blk, :, off] = outer
        elif kv.fp8:
            kq, ks = ref.quant_kv_token_head(k, kv.k_static)
            vq, vs = ref.quant_kv_token_head(v, kv.v_static)
            kv.k[blk, :, off] = kq
            kv.v[blk, :, off] = vq
            if kv.k_scale is not None:
                kv.k_scale[blk, :, off] = ks
                kv.v_scale[blk, :, off] = vs
        else:
            kv.k[blk, :, off] = k.to(kv.k.dtype)
            kv.v[blk, :, off] = v.to(kv.v.dtype)
        return q.reshape(t, hq * hd).to(qkv.dtype)
    if rope_pos3 is not None:
        rc = _lib.kernels().sllm_rope_kv_append_mrope(
            _p(qkv), _p(positions), _p(seq_index), _p(block_table), block_table.stride(0), _p(kv.k), _p(kv.v),
            _p(kv.k_scale), _p(kv.v_scale), t, hq, hkv, hd, rd, kv.page_size, kv.mode, theta, kv.k_static,
            kv.v_static, _p(inv_freq), _p(rope_pos3), int(mrope_sections[0]), int(mrope_sections[1]), _stream())
        _lib.check(rc, "rope_kv_append_mrope")
        return qkv[:, :hq * hd]
    if pair_offset > 0:
        rc = _lib.kernels().sllm_rope_kv_append_paired(
            _p(qkv), _p(positions), _p(seq_index), _p(block_table), block_table.stride(0), _p(kv.k), _p(kv.v),
            _p(kv.k_scale), _p(kv.v_scale), t, hq, hkv, hd, rd, kv.page_size, kv.mode, theta, kv.k_static,
            kv.v_static, _p(inv_freq), pair_offset, _stream())
        _lib.check(rc, "rope_kv_append_paired")
        return qkv[:, :hq * hd]
    rc = _lib.kernels().sllm_rope_kv_append(
        _p(qkv), _p(positions), _p(seq_index), _p(block_table), block_table.stride(0), _p(kv.k), _p(kv.v),
        _p(kv.k_scale), _p(kv.v_scale), t, hq, hkv, hd, rd, kv.page_size, kv.mode, theta, kv.k_static,
        kv.v_static, _p(inv_freq), _stream())
    _lib.check(rc, "rope_kv_append")
    return qkv[:, :hq * hd]


def _attn_splits(rows: int, hkv: int, max_kv: int) -> int:
    """KV splits so that about 8 CTAs (32 warps) per SM are in flight: the kernel hides its
    load -> compute -> load chains with occupancy, and each split keeps >= 128 keys."""
    ctas = rows * hkv
    target = 8 * _SM_COUNT
    if ctas >= target or max_kv <= 128:
        return 1
    return max(1, min((target + ctas - 1) // ctas, (max_kv + 127) // 128, 64))


def paged_attention(q: torch.Tensor, kv: KVLayer, block_table: torch.Tensor, seq_index: torch.Tensor,
                    kv_lens: torch.Tensor, hq: int, hkv: int, hd: int, *, window: int = 0,
                    sm_scale: Optional[float] = None, max_kv: int = 0, quant_out: bool = False,
                    sinks: Optional[torch.Tensor] = None, impl: Optional[str] = None, out: Optional[QTensor] = None):
    """Attention of each query row over its sequence's pages. q: [R, hq*hd] (row stride allowed).
    Returns [R, hq*hd] (bf16) or a QTensor when quant_out (head_dim 128); ``out`` supplies the QTensor to fill
    (its scale plane may have a leading dimension larger than R)."""
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(hd)
    r = q.shape[0]
    if _lib.on_cpu(q):
        out = torch.empty((r, hq, hd), dtype=torch.float32)
        for i in range(r):
            s = int(seq_index[i])
            n = int(kv_lens[i])
            nblk = (n + kv.page_size - 1) // kv.page_size
            blks = block_table[s, :nblk].long()
            if kv.nvfp4:
                kk = ref.dequant_kv_nvfp4_rows(kv.k[blks], kv.k_scale[blks], hd).transpose(1, 2).reshape(-1, hkv, hd)
                vv = ref.dequant_kv_nvfp4_rows(kv.v[blks], kv.v_scale[blks], hd).transpose(1, 2).reshape(-1, hkv, hd)
            elif kv.fp8:
                kk = ref.from_e4m3(kv.k[blks]).transpose(1, 2).reshape(-1, hkv, hd)
                vv = ref.from_e4m3(kv.v[blks]).transpose(1, 2).reshape(-1, hkv, hd)
                if kv.k_scale is not None:
                    kk = kk * kv.k_scale[blks].transpose(1, 2).reshape(-1, hkv, 1)
                    vv = vv * kv.v_scale[blks].transpose(1, 2).reshape(-1, hkv, 1)
                else:
                    kk, vv = kk * kv.k_static, vv * kv.v_static
            else:
                kk = kv.k[blks].transpose(1, 2).reshape(-1, hkv, hd).to(torch.float32)
                vv = kv.v[blks].transpose(1, 2).reshape(-1, hkv, hd).to(torch.float32)
            out[i] = ref.attention_rows(q[i].view(hq, hd), kk, vv, n, window, scale, sinks)
        out = out.view(r, hq * hd)
        if q.dtype == torch.float32 and not quant_out:
            return out
        out = ref.round_bf16(out)
        return QTensor(*ref.quant_fp8_1x128(out)) if quant_out else out.to(q.dtype)
    lib = _lib.kernels()
    wsp = workspace(q.device)
    splits = _attn_splits(r, hkv, max_kv if max_kv > 0 else block_table.shape[1] * kv.page_size)
    if quant_out:
        if hd != 128:
            raise ValueError("quantised attention output needs head_dim 128")
        oq = out if out is not None else _alloc_q(r, hq * hd, q.device)
        out_b, out_q, out_s, ld = None, oq.data, oq.scale, max(oq.scale.stride(0), oq.scale.shape[1])
    else:
        ob = torch.empty((r, hq * hd), dtype=torch.bfloat16, device=q.device)
        out_b, out_q, out_s, ld = ob, None, None, 0
    use_tc = (kv.fp8 and hd == 128 and (hq // hkv) in (1, 2, 4, 8, 16) and 128 % kv.page_size == 0
              and kv.page_size >= 8 and impl != "cuda_core")
    if impl == "tensor_core" and not use_tc:
        raise ValueError("tensor-core decode attention needs FP8 pages, head_dim 128 and a GQA group <= 16")
    if use_tc:
        mk = max_kv if max_kv > 0 else block_table.shape[1] * kv.page_size
        ctas = r * hkv
        # one wave of 2 CTAs per SM; a split keeps at least one 128-key tile
        splits = max(1, min((2 * _SM_COUNT) // ctas, (mk + 127) // 128, 64)) if ctas < 2 * _SM_COUNT else 1
        if _lib.audit_enabled():
            _lib.record_dispatch("paged_attention", "decode_attention_tc_kernel", rows=r, hq=hq, hkv=hkv, hd=hd, window=window,
                                 splits=splits, grid=[r, hkv, splits])
        rc = lib.sllm_decode_attention_tc(
            _p(q), q.stride(0), _p(kv.k), _p(kv.v), _p(kv.k_scale), _p(kv.v_scale), kv.k_static, kv.v_static,
            _p(block_table), block_table.stride(0), _p(seq_index), _p(kv_lens), r, hq, hkv, kv.k.shape[0],
            kv.page_size, window, scale, _p(out_b), _p(out_q), _p(out_s), ld, _p(sinks), splits, _p(wsp.ws),
            wsp.ws.numel(), _p(wsp.counters), wsp.counters.numel(), _p(wsp.status), _stream())
        _lib.check(rc, "decode_attention_tc")
        return oq if quant_out else ob
    if _lib.audit_enabled():
        # the CUDA-core kernel serves what the tensor-core kernel does not cover; for FP8 pages of 128-wide heads
        # that is a detour worth seeing
        _lib.record_dispatch("paged_attention", "paged_attention_kernel", fallback_used=bool(kv.fp8 and hd == 128),
                             rows=r, hq=hq, hkv=hkv, hd=hd, window=window, splits=splits)
    rc = lib.sllm_paged_attention(
        _p(q), q.stride(0), _p(kv.k), _p(kv.v), _p(kv.k_scale), _p(kv.v_scale), kv.k_static, kv.v_static,
        _p(block_table), block_table.stride(0), _p(seq_index), _p(kv_lens), r, hq, hkv, hd, kv.page_size, window,
        scale, kv.mode, _p(out_b), _p(out_q), _p(out_s), ld, _p(sinks), splits, _p(wsp.ws), wsp.ws.numel(),
        _p(wsp.counters), wsp.counters.numel(), _stream())
    _lib.check(rc, "paged_attention")
    return oq if quant_out else ob

"""4-bit block-scaled weights (MXFP4 / NVFP4): resident layout, the tcgen05 W4A16 GEMM and its CPU oracle.

File formats keep the layouts of the reference (codes: low nibble = even element; MXFP4 scales E8M0
[N, K/32]; NVFP4 scales E4M3 [N, K/16] plus an FP32 tensor scale - docs/quantization/nvfp4.md:18-31,
docs/formats/gguf.md:40-41).  `W4Weight.from_file_layout` repacks them once at load into what the kernel
streams: rows padded to 128 and K to 128, nibbles of every eight elements reordered to
(e0,e2,e4,e6,e1,e3,e5,e7), and codes and scales tiled together as
[group][row tile][K chunk]{128 rows x 64 B codes | 128 rows x (4|8) B scales} so that one CTA reads one
contiguous stretch of HBM with a single bulk copy per chunk.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from ..formats import codecs
from . import _lib

MAX_E8M0_CODE = 144


@dataclass
class W4Weight:
    fmt: str                    # mxfp4 | nvfp4
    groups: int
    n: int                      # output features per group
    k: int                      # input features
    n_rows: int                 # n padded to 128
    k_pad: int                  # k padded to 128
    tiles: torch.Tensor         # uint8 [groups, n_rows / 128, k_pad / 128, 8192 + 128 * (4 | 8)]
    tensor_scale: Optional[torch.Tensor]   # fp32 [groups] (nvfp4)
    file_packed: Optional[np.ndarray] = None    # kept on CPU weights for the oracle
    file_scales: Optional[np.ndarray] = None
    native: Optional[torch.Tensor] = None       # tiles of the block-scaled tensor-core path (see `native_tiles`)

    @property
    def block(self) -> int:
        return 32 if self.fmt == "mxfp4" else 16

    @staticmethod
    def from_file_layout(fmt: str, packed: np.ndarray, scales: np.ndarray, k: int, tensor_scale=None,
                         device="cpu", keep_file: bool = False) -> "W4Weight":
        """packed: uint8 [G, N, ceil(K/2)] (or [N, ...]); scales: uint8 [G, N, ceil(K/block)]."""
        if packed.ndim == 2:
            packed, scales = packed[None], scales[None]
        g, n, kb = packed.shape
        block = 32 if fmt == "mxfp4" else 16
        sb = 128 // block
        if fmt == "mxfp4" and int(scales.max(initial=0)) > MAX_E8M0_CODE:
            raise ValueError("MXFP4 block scale above 2^17 is outside the kernel's exact range")
        n_rows, k_pad = (n + 127) // 128 * 128, (k + 127) // 128 * 128
        codes = np.zeros((g, n_rows, k_pad), dtype=np.uint8)
        codes[:, :n, :k] = codecs.unpack_nibbles(packed, k)
        c8 = codes.reshape(g, n_rows, k_pad // 8, 8)
        order = [0, 2, 4, 6, 1, 3, 5, 7]                 # nibble position p holds element order[p]
        re = c8[..., order]
        words = np.zeros(re.shape[:-1], dtype=np.uint32)
        for pos in range(8):
            words |= re[..., pos].astype(np.uint32) << (4 * pos)
        rt, kc = n_rows // 128, k_pad // 128
        res_packed = words.view(np.uint8).reshape(g, rt, 128, kc, 64).transpose(0, 1, 3, 2, 4).reshape(g, rt, kc, 8192)
        sc = np.zeros((g, n_rows, k_pad // block), dtype=np.uint8)
        sc[:, :n, :scales.shape[2]] = scales
        sc_t = sc.reshape(g, rt, 128, kc, sb).transpose(0, 1, 3, 2, 4).reshape(g, rt, kc, 128 * sb)
        tiled = np.concatenate([res_packed, sc_t], axis=3)
        ts = None
        if fmt == "nvfp4":
            tsv = np.ones(g, dtype=np.float32) if tensor_scale is None else np.asarray(tensor_scale, dtype=np.float32).reshape(g)
            ts = torch.from_numpy(tsv.copy()).to(device)
        return W4Weight(fmt, g, n, k, n_rows, k_pad, torch.from_numpy(np.ascontiguousarray(tiled)).to(device), ts,
                        packed.copy() if keep_file else None, scales.copy() if keep_file else None)

    @staticmethod
    def quantize(fmt: str, w: torch.Tensor, device="cpu", keep_file: bool = True) -> "W4Weight":
        """w: float [G, N, K] or [N, K]."""
        w3 = w.float().cpu().numpy()
        if w3.ndim == 2:
            w3 = w3[None]
        pk, sc, ts = [], [], []
        for gi in range(w3.shape[0]):
            if fmt == "mxfp4":
                p, s = codecs.quantize_mxfp4(w3[gi])
            else:
                p, s, t = codecs.quantize_nvfp4(w3[gi])
                ts.append(t)
            pk.append(p)
            sc.append(s)
        return W4Weight.from_file_layout(fmt, np.stack(pk), np.stack(sc), w3.shape[2], ts or None, device, keep_file)

    @staticmethod
    def quantize_device(fmt: str, w: torch.Tensor) -> "W4Weight":
        """Same quantiser as `quantize`, written in torch ops so that it runs on the GPU (benchmark-sized random
        weights); w: float/bf16 [G, N, K] or [N, K] on any device.  Bit-identical to the NumPy codec."""
        if w.dim() == 2:
            w = w[None]
        if w.shape[0] > 1 and w.numel() > (1 << 27):
            # large expert stacks: quantise a few groups at a time to bound the temporaries
            step = max(1, (1 << 27) // (w.shape[1] * w.shape[2]))
            parts = [W4Weight.quantize_device(fmt, w[i:i + step]) for i in range(0, w.shape[0], step)]
            p0 = parts[0]
            ts = None if p0.tensor_scale is None else torch.cat([p.tensor_scale for p in parts])
            return W4Weight(fmt, w.shape[0], p0.n, p0.k, p0.n_rows, p0.k_pad, torch.cat([p.tiles for p in parts]), ts)
        dev = w.device
        g, n, k = w.shape
        block = 32 if fmt == "mxfp4" else 16
        sb = 128 // block
        n_rows, k_pad = (n + 127) // 128 * 128, (k + 127) // 128 * 128
        wf = torch.zeros((g, n_rows, k_pad), dtype=torch.float32, device=dev)
        wf[:, :n, :k] = w.float()
        blk = wf.view(g, n_rows, k_pad // block, block)
        bamax = torch.where(torch.isfinite(blk), blk.abs(), torch.zeros_like(blk)).amax(dim=3)
        ts = None
        if fmt == "mxfp4":
            bits = bamax.contiguous().view(torch.int32).to(torch.int64) + 0x00200000
            code = (((bits & 0x7F800000) >> 23) - 2).clamp(0, 254)
            code = torch.where(bamax == 0, torch.zeros_like(code), code)
            if int(code.max()) > MAX_E8M0_CODE:
                raise ValueError("MXFP4 block scale above 2^17 is outside the kernel's exact range")
            scale = torch.ldexp(torch.ones_like(bamax), (code - 127).to(torch.int32))
            sc_codes = code.to(torch.uint8)
        else:
            amax = bamax.view(g, -1).amax(dim=1)
            ts = torch.where(amax > 0, amax / (448.0 * 6.0), torch.ones_like(amax)).float()
            want = (bamax / 6.0) / ts.view(g, 1, 1)
            sc_codes = want.clamp(max=448.0).to(torch.float8_e4m3fn).view(torch.uint8)
            scale = sc_codes.view(torch.float8_e4m3fn).float() * ts.view(g, 1, 1)
        safe = torch.where(scale > 0, scale, torch.ones_like(scale))
        a = (blk / safe.unsqueeze(-1)).abs().clamp(max=6.0)
        vals = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], device=dev)
        hi = torch.bucketize(a, vals).clamp(max=7)             # first index with vals[hi] >= a
        lo = (hi - 1).clamp(min=0)
        dlo, dhi = (a - vals[lo]).abs(), (vals[hi] - a).abs()
        pick_hi = (dhi < dlo) | ((dhi == dlo) & ((hi & 1) == 0))
        idx = torch.where(pick_hi, hi, lo)
        sign = ((blk < 0) & (idx != 0)).to(torch.int64) << 3
        codes = (idx | sign)
        codes = torch.where((scale > 0).unsqueeze(-1), codes, torch.zeros_like(codes)).view(g, n_rows, k_pad // 8, 8)
        order = [0, 2, 4, 6, 1, 3, 5, 7]
        words = torch.zeros((g, n_rows, k_pad // 8), dtype=torch.int64, device=dev)
        for pos in range(8):
            words |= codes[..., order[pos]] << (4 * pos)
        words = torch.where(words >= (1 << 31), words - (1 << 32), words).to(torch.int32)
        rt, kc = n_rows // 128, k_pad // 128
        pk = words.view(torch.uint8).view(g, rt, 128, kc, 64).permute(0, 1, 3, 2, 4).reshape(g, rt, kc, 8192)
        sc_t = sc_codes.view(g, rt, 128, kc, sb).permute(0, 1, 3, 2, 4).reshape(g, rt, kc, 128 * sb)
        tiles = torch.cat([pk, sc_t], dim=3).contiguous()
        return W4Weight(fmt, g, n, k, n_rows, k_pad, tiles, ts)

    def dequantized(self, group: int = 0) -> torch.Tensor:
        """fp32 [n, k] of one group from the resident layout (exact)."""
        rt, kc = self.n_rows // 128, self.k_pad // 128
        t = self.tiles.cpu().numpy()[group]
        pk = np.ascontiguousarray(t[:, :, :8192].reshape(rt, kc, 128, 64).transpose(0, 2, 1, 3)).reshape(self.n_rows, self.k_pad // 2)
        words = pk.view(np.uint32).reshape(self.n_rows, self.k_pad // 8)
        order = [0, 2, 4, 6, 1, 3, 5, 7]
        codes = np.zeros((self.n_rows, self.k_pad // 8, 8), dtype=np.uint8)
        for pos in range(8):
            codes[..., order[pos]] = (words >> (4 * pos)) & 0xF
        vals = codecs.decode_e2m1(codes.reshape(self.n_rows, self.k_pad))
        sb = 128 // self.block
        sc = t[:, :, 8192:].reshape(rt, kc, 128, sb).transpose(0, 2, 1, 3).reshape(self.n_rows, self.k_pad // self.block)
        s = codecs.decode_e8m0(sc) if self.fmt == "mxfp4" else codecs.decode_e4m3fn(sc)
        if self.tensor_scale is not None:
            s = s * np.float32(float(self.tensor_scale[group].item()))
        out = vals * np.repeat(s, self.block, axis=1)
        return torch.from_numpy(out[:self.n, :self.k].astype(np.float32))

    def to_file_layout(self, group: int = 0):
        """(packed [n, k / 2] adjacent-pair nibbles, scales [n, k / block]) of one group: the inverse of
        ``from_file_layout`` (exact), used when a resident weight is written back to a model file."""
        rt, kc = self.n_rows // 128, self.k_pad // 128
        t = self.tiles.cpu().numpy()[group]
        pk = np.ascontiguousarray(t[:, :, :8192].reshape(rt, kc, 128, 64).transpose(0, 2, 1, 3)).reshape(self.n_rows, self.k_pad // 2)
        words = pk.view(np.uint32).reshape(self.n_rows, self.k_pad // 8)
        order = [0, 2, 4, 6, 1, 3, 5, 7]
        codes = np.zeros((self.n_rows, self.k_pad // 8, 8), dtype=np.uint8)
        for pos in range(8):
            codes[..., order[pos]] = (words >> (4 * pos)) & 0xF
        codes = codes.reshape(self.n_rows, self.k_pad)[:self.n, :self.k]
        sb = 128 // self.block
        sc = t[:, :, 8192:].reshape(rt, kc, 128, sb).transpose(0, 2, 1, 3).reshape(self.n_rows, self.k_pad // self.block)
        return codecs.pack_nibbles(codes), np.ascontiguousarray(sc[:self.n, :(self.k + self.block - 1) // self.block])

    def nbytes(self) -> int:
        return self.tiles.numel() + (self.native.numel() if self.native is not None else 0)

    def native_tiles(self) -> torch.Tensor:
        """Tiles for the W4A4 kernel (csrc/gemm_fp4.cu), built once from the resident ones on their device:
        uint8 [groups, row tiles, K blocks of 256, 16384 + 512 * atoms].  A tile is the 128-byte-swizzled shared-memory
        image of 128 rows x 128 B of codes in the standard nibble order (element 2 i in the low nibble of byte i),
        followed by the block's scale atoms (4 for block 16, 2 for block 32): 512 bytes = [32 r][4 j][4 s] holding scale s
        of row r + 32 j, the form tcgen05.cp moves to TMEM."""
        if self.native is not None:
            return self.native
        t = self.tiles
        g, rt, kc, _ = t.shape
        sb = 128 // self.block
        kb = (kc + 1) // 2
        dev = t.device
        rr = (torch.arange(128, device=dev) & 7).view(128, 1)
        src = (torch.arange(8, device=dev).view(1, 8) ^ rr).view(1, 1, 1, 128, 8, 1)
        out = torch.empty((g, rt, kb, 16384 + 128 * 2 * sb), dtype=torch.uint8, device=dev)
        step = max(1, (1 << 24) // max(1, rt * kc * 128 * 16))
        for g0 in range(0, g, step):
            tt = t[g0:g0 + step]
            gg = tt.shape[0]
            if kc % 2:
                tt = torch.cat([tt, torch.zeros((gg, rt, 1, tt.shape[3]), dtype=torch.uint8, device=dev)], dim=2)
            words = tt[..., :8192].contiguous().view(torch.int32).view(gg, rt, 2 * kb, 128, 16).to(torch.int64) & 0xFFFFFFFF
            # resident nibble order (e0,e2,e4,e6,e1,e3,e5,e7) -> bytes (e1 e0), (e3 e2), (e5 e4), (e7 e6)
            by = torch.stack([((words >> (4 * b)) & 0xF) | (((words >> (16 + 4 * b)) & 0xF) << 4) for b in range(4)],
                             dim=-1).to(torch.uint8)
            rows = by.view(gg, rt, kb, 2, 128, 64).permute(0, 1, 2, 4, 3, 5).reshape(gg, rt, kb, 128, 8, 16)
            img = torch.gather(rows, 4, src.expand(gg, rt, kb, 128, 8, 16)).reshape(gg, rt, kb, 16384)
            sc = tt[..., 8192:].reshape(gg, rt, kb, 2, 128, sb).permute(0, 1, 2, 4, 3, 5).reshape(gg, rt, kb, 4, 32, 2 * sb // 4, 4)
            atoms = sc.permute(0, 1, 2, 5, 4, 3, 6).reshape(gg, rt, kb, 128 * 2 * sb)
            out[g0:g0 + gg] = torch.cat([img, atoms], dim=3)
        self.native = out
        return out


@dataclass
class Fp4Act:
    """Activations already quantised for the W4A4 kernel (what `act_quant_fp4` returns), passed where a bf16 matrix
    would be: `ops.linear` / `linear_w4` / the tensor-parallel row-parallel projection accept it for 4-bit weights."""
    data: torch.Tensor          # codes uint8 [T, K_pad / 2]
    sf: torch.Tensor            # block scales, 8 bytes per four
    outer: torch.Tensor         # fp32 [T]
    k: int
    fmt: str

    @property
    def shape(self):
        return (self.data.shape[0], self.k)


def _bn_for(tokens: int) -> int:
    return 16 if tokens <= 16 else 32 if tokens <= 32 else 64 if tokens <= 64 else 128


def linear_w4(x: torch.Tensor, w: W4Weight, residual: Optional[torch.Tensor] = None, tok_off: Optional[torch.Tensor] = None,
              tok_scale: Optional[torch.Tensor] = None, max_group_tokens: Optional[int] = None, splits: int = 0,
              row_ptr: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """y[t, :] = x[t, :] @ W_g(t)^T (* tok_scale[t]) (+ residual).  Dense when tok_off is None (groups must be 1);
    grouped otherwise: tokens of group g are rows tok_off[g] .. tok_off[g + 1] of x."""
    if isinstance(x, Fp4Act):
        if x.k != w.k or x.fmt != w.fmt:
            raise ValueError("quantised activations do not match the weight's width or format")
        return linear_w4a4(None, w, residual, tok_off, tok_scale, max_group_tokens, 0, row_ptr,
                           quantized=(x.data, x.sf, x.outer))
    t, k = x.shape
    if k != w.k:
        raise ValueError("input width does not match the weight")
    if _lib.on_cpu(x):
        if w4a4_enabled() and x.dtype == torch.bfloat16 and k % 8 == 0 and (tok_off is not None or t <= W4A4_MAX_DENSE_ROWS):
            return linear_w4a4(x, w, residual, tok_off, tok_scale, max_group_tokens, 0, row_ptr)
        out = torch.zeros((t, w.n), dtype=torch.float32)
        offs = [0, t] if tok_off is None else tok_off.tolist()
        xf = x.float()
        for g in range(w.groups):
            a, b = offs[g], offs[g + 1]
            if b > a:
                out[a:b] = xf[a:b] @ w.dequantized(g).t()
        if tok_scale is not None:
            out = out * tok_scale.float()[:, None]
        if residual is not None:
            out = out + residual.float()
        return out if x.dtype == torch.float32 else out.to(torch.bfloat16)
    # 4-bit activations serve the decode regime (few rows per weight tile); a prompt's rows are compute bound and keep
    # bf16 activations on the W4A16 kernel
    if w4a4_enabled() and x.dtype == torch.bfloat16 and k % 8 == 0 and (tok_off is not None or t <= W4A4_MAX_DENSE_ROWS):
        return linear_w4a4(x, w, residual, tok_off, tok_scale, max_group_tokens, 0, row_ptr)
    from .core import _p, _stream, workspace
    P, I, L, F = C.c_void_p, C.c_int, C.c_longlong, C.c_float
    _lib.EXTRA_KERNEL_SIGNATURES.setdefault("sllm_gemm_w4", (I, [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, I,
                                                               P, L, P, I, P, P]))
    if w.groups > 1 and tok_off is None:
        raise ValueError("grouped weights need token offsets")
    x = x.contiguous() if x.stride(1) != 1 or x.stride(0) % 8 else x
    y = torch.empty((t, w.n), dtype=torch.bfloat16, device=x.device)
    mgt = max_group_tokens or t
    bn = _bn_for(mgt if tok_off is None else min(mgt, 32))
    k_chunks = w.k_pad // 128
    if splits <= 0:
        ctas = (w.n_rows // 128) * (w.groups if tok_off is None else max(1, min(w.groups, t))) * ((min(mgt, t) + bn - 1) // bn)
        splits = 1
        while ctas * splits < 148 and splits * 2 <= max(1, k_chunks // 4) and splits < 16:
            splits *= 2
    wsp = workspace(x.device)
    if _lib.audit_enabled():
        _lib.record_dispatch("linear_w4", "gemm_w4_kernel", fmt=w.fmt, tokens=t, n=w.n, k=w.k, groups=w.groups,
                             grouped=tok_off is not None, bn=bn, splits=splits)
    if row_ptr is not None:
        # scatter epilogue: result row t goes to the bf16 row at address row_ptr[t] (int64, may be peer memory)
        if residual is not None or row_ptr.dtype != torch.int64 or row_ptr.numel() < t:
            raise ValueError("row_ptr: int64 addresses, one per token row, and no residual")
        _lib.EXTRA_KERNEL_SIGNATURES.setdefault("sllm_gemm_w4_scatter", (I, [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I,
                                                                           I, P, L, P, I, P, P]))
        rc = _lib.kernels().sllm_gemm_w4_scatter(_p(w.tiles), _p(w.tensor_scale), _p(x), _p(row_ptr), _p(tok_off),
                                                 _p(tok_scale), 0 if w.fmt == "mxfp4" else 1, w.groups, w.n_rows, w.n, w.k_pad,
                                                 w.k, x.stride(0), t, mgt, bn, splits, 0, _p(wsp.ws), wsp.ws.numel(),
                                                 _p(wsp.counters), wsp.counters.numel(), _p(wsp.status), _stream())
        _lib.check(rc, "gemm_w4_scatter")
        return None
    rc = _lib.kernels().sllm_gemm_w4(_p(w.tiles), _p(w.tensor_scale), _p(x), _p(y), _p(residual), _p(tok_off),
                                     _p(tok_scale), 0 if w.fmt == "mxfp4" else 1, w.groups, w.n_rows, w.n, w.k_pad, w.k,
                                     x.stride(0), t, mgt, y.stride(0), bn, splits, 0, _p(wsp.ws), wsp.ws.numel(),
                                     _p(wsp.counters), wsp.counters.numel(), _p(wsp.status), _stream())
    _lib.check(rc, "gemm_w4")
    return y


# ------------------------------------------------------------------------------------------ W4A4 (block-scaled MMA)
_W4A4 = {"on": None}


def w4a4_enabled() -> bool:
    """Whether 4-bit GEMMs quantise their activations to the weights' own 4-bit format and run on the block-scaled
    tensor-core path (SLLM_W4A4=1 or `set_w4a4(True)`); off by default: W4A16 is the accuracy baseline."""
    if _W4A4["on"] is None:
        import os
        _W4A4["on"] = os.environ.get("SLLM_W4A4", "0") == "1"
    return _W4A4["on"]


def set_w4a4(on: bool) -> None:
    _W4A4["on"] = bool(on)


def act_quant_fp4(x: torch.Tensor, fmt: str, src_row: Optional[torch.Tensor] = None, tokens: Optional[int] = None,
                  n_rows: Optional[torch.Tensor] = None, gated: Optional[str] = None, norm: Optional[tuple] = None):
    """bf16 [T, K] -> (codes uint8 [T, K_pad / 2], block scales uint8 [T, 2 K_pad / block], row scales fp32 [T]) with K
    padded to 256.  The scale matrix is the kernel's operand: four scale bytes, then four unused ones (`sf_compact`
    drops them).  nvfp4: row scale amax / 2688, UE4M3 block scales; mxfp4: UE8M0 block scales, row scale 1.
    `src_row` (int32 [T]): token t reads row src_row[t] of x; `n_rows` (int32 device scalar): tokens from *n_rows on are
    skipped (their outputs stay undefined); `gated` ("silu" | "gelu_tanh"): x is [T, 2 K] = [gate | up] and
    act(gate) * up is what gets quantised; `norm` = (weight bf16 [K], eps, offset_one): the RMS-normalised row is what
    gets quantised (not together with `gated`)."""
    from . import reference
    t = tokens if tokens is not None else (x.shape[0] if src_row is None else src_row.numel())
    k = x.shape[1] // 2 if gated else x.shape[1]
    block = 32 if fmt == "mxfp4" else 16
    k_pad = (k + 255) // 256 * 256
    if _lib.on_cpu(x):
        xs = x if src_row is None else x.index_select(0, src_row.long()[:t].clamp(0, x.shape[0] - 1))
        xs = xs[:t]
        if gated:
            xs = reference.round_bf16(reference.gated_act(xs, gated))
        if norm is not None:
            xs = reference.round_bf16(reference.rmsnorm(xs, norm[0], norm[1], norm[2]))
        codes, sf, outer = reference.quant_act_fp4(xs, fmt)
        return codes, sf_padded(sf), outer
    from .core import _p, _stream
    P, I = C.c_void_p, C.c_int
    _lib.EXTRA_KERNEL_SIGNATURES.setdefault("sllm_act_quant_fp4", (I, [P, I, I, I, I, P, P, I, P, C.c_float, I, I, P, P, I, P, P]))
    if norm is not None and (gated or norm[0].dtype != torch.bfloat16 or norm[0].numel() != k):
        raise ValueError("act_quant_fp4: norm takes a bf16 weight of the row width and excludes gated")
    if x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.stride(0) % 8 or k % 8:
        raise ValueError("act_quant_fp4: bf16 rows with a stride and width that are multiples of 8")
    xq = torch.empty((t, k_pad // 2), dtype=torch.uint8, device=x.device)
    xsf = torch.empty((t, 2 * k_pad // block), dtype=torch.uint8, device=x.device)      # a multiple of 16 bytes
    outer = torch.empty((t,), dtype=torch.float32, device=x.device)
    g = 0 if not gated else 1 if gated == "silu" else 2
    nw, eps, off1 = (norm[0], float(norm[1]), int(bool(norm[2]))) if norm is not None else (None, 0.0, 0)
    rc = _lib.kernels().sllm_act_quant_fp4(_p(x), x.stride(0), t, k, k_pad, _p(src_row), _p(n_rows), g, _p(nw), eps, off1,
                                           0 if fmt == "mxfp4" else 1, _p(xq), _p(xsf), xsf.stride(0), _p(outer), _stream())
    _lib.check(rc, "act_quant_fp4")
    return xq, xsf, outer


def sf_padded(sf: torch.Tensor) -> torch.Tensor:
    """Compact block scales [T, n] -> the kernel's operand [T, 2 n]: every four scale bytes followed by four zeros."""
    t, n = sf.shape
    out = torch.zeros((t, n // 4, 8), dtype=torch.uint8, device=sf.device)
    out[:, :, :4] = sf.view(t, n // 4, 4)
    return out.view(t, 2 * n)


def sf_compact(xsf: torch.Tensor) -> torch.Tensor:
    t, n = xsf.shape
    return xsf.view(t, n // 8, 8)[:, :, :4].reshape(t, n // 2)


W4A4_MAX_DENSE_ROWS = 32


def linear_w4a4(x: torch.Tensor, w: W4Weight, residual: Optional[torch.Tensor] = None, tok_off: Optional[torch.Tensor] = None,
                tok_scale: Optional[torch.Tensor] = None, max_group_tokens: Optional[int] = None, splits: int = 0,
                row_ptr: Optional[torch.Tensor] = None, quantized=None, bn: Optional[int] = None) -> Optional[torch.Tensor]:
    """`linear_w4` with the activations quantised to the weights' 4-bit format first (or passed as `quantized` =
    (codes, block scales, row scales) from `act_quant_fp4`).  The tensor core multiplies E2M1 by E2M1 and applies both
    block scales; the row and tensor scales are applied to the fp32 sums.  Token tiles are 16 or 32 rows wide (the
    weights of a row tile are streamed once per token tile: the decode and routed-expert regime); `bn` = 64 / 128
    selects the wide tiles, whose K range per CTA is bounded (split-K through the workspace)."""
    t, k = x.shape if quantized is None else (quantized[0].shape[0], w.k)
    if k != w.k:
        raise ValueError("input width does not match the weight")
    q = quantized if quantized is not None else act_quant_fp4(x, w.fmt)
    xq, xsf, outer = q
    if _lib.on_cpu(xq):
        from . import reference
        xf = reference.dequant_act_fp4(xq, sf_compact(xsf), outer, w.fmt)[:, :k]
        out = torch.zeros((t, w.n), dtype=torch.float32)
        offs = [0, t] if tok_off is None else tok_off.tolist()
        for g in range(w.groups):
            a, b = offs[g], offs[g + 1]
            if b > a:
                out[a:b] = xf[a:b] @ w.dequantized(g).t()
        if tok_scale is not None:
            out = out * tok_scale.float()[:, None]
        if residual is not None:
            out = out + residual.float()
        return out.to(torch.bfloat16)
    from .core import _p, _stream, workspace
    P, I, L = C.c_void_p, C.c_int, C.c_longlong
    _lib.EXTRA_KERNEL_SIGNATURES.setdefault("sllm_gemm_fp4", (I, [P, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I,
                                                                P, L, P, I, P, P]))
    if w.groups > 1 and tok_off is None:
        raise ValueError("grouped weights need token offsets")
    tiles = w.native_tiles()
    kb = tiles.shape[2]
    mgt = max_group_tokens or t
    if bn is None:
        bn = _bn_for(min(mgt, 32))
    min_splits = (kb + 7) // 8 if bn > 32 else 1
    if splits <= 0:
        ctas = (w.n_rows // 128) * (w.groups if tok_off is None else max(1, min(w.groups, t))) * ((min(mgt, t) + bn - 1) // bn)
        splits = min_splits
        if bn > 32:
            while ctas * splits < 148 and splits * 2 <= max(1, kb // 2) and splits < 16:
                splits *= 2
        elif ctas < 100 and kb >= 64:
            # decode tiles: a K split costs more than it balances (measured: one split wins down to 80 row tiles);
            # only a long K over few row tiles is worth two
            splits = 2
    splits = max(splits, min_splits)
    wsp = workspace(xq.device)
    if _lib.audit_enabled():
        _lib.record_dispatch("linear_w4a4", "gemm_fp4_kernel", fmt=w.fmt, tokens=t, n=w.n, k=w.k, groups=w.groups,
                             grouped=tok_off is not None, bn=bn, splits=splits)
    y = None
    if row_ptr is None:
        y = torch.empty((t, w.n), dtype=torch.bfloat16, device=xq.device)
    elif residual is not None or row_ptr.dtype != torch.int64 or row_ptr.numel() < t:
        raise ValueError("row_ptr: int64 addresses, one per token row, and no residual")
    rc = _lib.kernels().sllm_gemm_fp4(_p(tiles), _p(w.tensor_scale), _p(xq), _p(xsf), xsf.stride(0), _p(outer), _p(y),
                                      _p(residual), _p(tok_off), _p(tok_scale), _p(row_ptr), 0 if w.fmt == "mxfp4" else 1,
                                      w.groups, w.n_rows, w.n, kb * 256, t, mgt, w.n, bn, splits, _p(wsp.ws), wsp.ws.numel(),
                                      _p(wsp.counters), wsp.counters.numel(), _p(wsp.status), _stream())
    _lib.check(rc, "gemm_fp4")
    return y

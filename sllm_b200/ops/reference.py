"""Plain PyTorch restatements of every op, computed in fp32 (or the input dtype on CPU).

They serve two purposes: the numerics oracle for the CUDA kernels in the tests, and the execution
path for CPU tensors (the tiny fp32 decoder used for token-for-token checks).  They mirror the
kernels' rounding points (bf16 round after norm / activation, E4M3 saturation, scale = amax / 448)
so that results are comparable within the stated tolerances.

Oracle lineage: tests/reference/oracles.py:22-142 (bf16 RNE, RMSNorm), ci/tools/verify_kv_lowbit_oracle.py
(low-bit KV) of the reference, restated from their documented maths.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

E4M3_MAX = 448.0


def round_bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32) if x.dtype != torch.bfloat16 else x.to(torch.float32)


def to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> E4M3FN bytes (uint8): RNE, saturate to +-448, NaN -> 0x7f."""
    xf = x.to(torch.float32)
    nan = torch.isnan(xf)
    q = xf.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)
    return torch.where(nan, torch.full_like(q, 0x7F), q)


def from_e4m3(b: torch.Tensor) -> torch.Tensor:
    return b.view(torch.float8_e4m3fn).to(torch.float32)


def quant_fp8_1x128(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """[M, K] -> (E4M3 bytes [M, K], scales [ceil(K/128), M] fp32)."""
    m, k = x.shape
    nkb = (k + 127) // 128
    xf = x.to(torch.float32)
    pad = nkb * 128 - k
    if pad:
        xf = torch.nn.functional.pad(xf, (0, pad))
    blk = xf.view(m, nkb, 128)
    finite = torch.where(torch.isfinite(blk), blk.abs(), torch.zeros_like(blk))
    amax = finite.amax(dim=-1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = to_e4m3(blk / scale.unsqueeze(-1)).view(m, nkb * 128)[:, :k].contiguous()
    return q, scale.t().contiguous()


def dequant_fp8_1x128(q: torch.Tensor, scale_t: torch.Tensor) -> torch.Tensor:
    m, k = q.shape
    s = scale_t.t().repeat_interleave(128, dim=1)[:, :k]
    return from_e4m3(q) * s


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, offset_one: bool = False) -> torch.Tensor:
    xf = x.to(torch.float32)
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    g = w.to(torch.float32)
    if offset_one:
        g = 1.0 + g
    return xf * inv * g


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.gelu(x, approximate="tanh")


def gated_act(x: torch.Tensor, act: str = "silu", round_intermediate: bool = True) -> torch.Tensor:
    inter = x.shape[-1] // 2
    g, u = x[..., :inter].to(torch.float32), x[..., inter:].to(torch.float32)
    a = silu(g) if act == "silu" else gelu_tanh(g)
    if round_intermediate:
        a = round_bf16(a)
    return a * u


def rope_split_half(x: torch.Tensor, positions: torch.Tensor, theta: float, rotary_dim: Optional[int] = None,
                    inv_freq: Optional[torch.Tensor] = None, rope_pos3: Optional[torch.Tensor] = None,
                    sections: Optional[tuple] = None, pair_offset: int = 0) -> torch.Tensor:
    """x: [T, H, D]; rotates the first rotary_dim channels, pairing channel i with i + rotary_dim/2.  With
    rope_pos3 [3, T] and sections (sec_t, sec_h), rotary pair j turns with the temporal index for j < sec_t, the
    height index for j < sec_t + sec_h and the width index otherwise.  ``pair_offset`` > 0 is the "proportional"
    layout: channel i < rotary_dim / 2 pairs with i + pair_offset (= D / 2), frequencies theta^(-2 i / D)."""
    t, h, d = x.shape
    r = rotary_dim or d
    half = r // 2
    poff = pair_offset if pair_offset > 0 else half
    xf = x.to(torch.float32)
    if inv_freq is None:
        inv_freq = theta ** (-2.0 * torch.arange(half, dtype=torch.float32, device=x.device) / (d if pair_offset > 0 else r))
    if rope_pos3 is not None:
        st, sh = sections
        axis = torch.tensor([0 if j < st else (1 if j < st + sh else 2) for j in range(half)], device=x.device)
        pos = rope_pos3.to(torch.float32).t()[:, axis]                                       # [T, half]
        ang = pos * inv_freq.to(torch.float32).unsqueeze(0)
    else:
        ang = positions.to(torch.float32).unsqueeze(-1) * inv_freq.to(torch.float32).unsqueeze(0)  # [T, half]
    cs, sn = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
    a, b = xf[..., :half], xf[..., poff:poff + half]
    out = xf.clone()
    out[..., :half] = a * cs - b * sn
    out[..., poff:poff + half] = b * cs + a * sn
    return out


def quant_kv_token_head(x: torch.Tensor, static_scale: float = 0.0) -> tuple[torch.Tensor, torch.Tensor]:
    """x: [T, H, D] -> (E4M3 bytes, scale [T, H]) with scale = amax / 448 per (token, head)."""
    xf = x.to(torch.float32)
    if static_scale > 0:
        scale = torch.full(xf.shape[:-1], static_scale, dtype=torch.float32, device=x.device)
    else:
        finite = torch.where(torch.isfinite(xf), xf.abs(), torch.zeros_like(xf))
        amax = finite.amax(dim=-1)
        scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    return to_e4m3(xf / scale.unsqueeze(-1)), scale


def attention_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kv_len: int, window: int, sm_scale: float,
                   sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One query row. q: [Hq, D]; k, v: [S, Hkv, D] (fp32, already dequantised); keys [first, kv_len)."""
    hq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    first = max(0, kv_len - window) if window > 0 else 0
    ks = k[first:kv_len].to(torch.float32).repeat_interleave(g, dim=1)  # [S', Hq, D]
    vs = v[first:kv_len].to(torch.float32).repeat_interleave(g, dim=1)
    s = torch.einsum("hd,shd->hs", q.to(torch.float32) * sm_scale, ks)
    if sink is not None:
        s = torch.cat([s, sink.to(torch.float32).view(hq, 1)], dim=1)
        p = torch.softmax(s, dim=-1)[:, :-1]
    else:
        p = torch.softmax(s, dim=-1)
    return torch.einsum("hs,shd->hd", p, vs)


def linear_fp8(xq: torch.Tensor, xs_t: torch.Tensor, wq: torch.Tensor, ws_t: torch.Tensor) -> torch.Tensor:
    """Block-scaled FP8 GEMM oracle: dequantise both sides, fp32 matmul. Returns fp32 [M, N]."""
    return dequant_fp8_1x128(xq, xs_t) @ dequant_fp8_1x128(wq, ws_t).t()


def sm_scale_default(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)


def quant_kv_nvfp4_rows(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """x: [T, H, D] -> (rows uint8 [T, H, D / 2 + D / 16] = E2M1 codes then E4M3 block scales, outer fp32 [T, H]):
    the NVFP4 KV row of the paged cache, through the host codec (formats.codecs.quantize_kv_nvfp4)."""
    from ..formats import codecs
    packed, bsc, outer = codecs.quantize_kv_nvfp4(x.to(torch.float32).cpu().numpy())
    import numpy as np
    rows = np.concatenate([packed, bsc], axis=-1)
    return torch.from_numpy(rows).to(x.device), torch.from_numpy(outer).to(x.device)


def dequant_kv_nvfp4_rows(rows: torch.Tensor, outer: torch.Tensor, d: int) -> torch.Tensor:
    """Inverse of quant_kv_nvfp4_rows for any leading shape: rows [..., D / 2 + D / 16], outer [...] -> fp32 [..., D]."""
    from ..formats import codecs
    import numpy as np
    r = rows.cpu().numpy()
    lead = r.shape[:-1]
    flat = r.reshape(-1, r.shape[-1])
    codes = codecs.unpack_nibbles(flat[:, :d // 2], d)
    bs = codecs.decode_e4m3fn(flat[:, d // 2:]) * outer.cpu().numpy().reshape(-1, 1).astype(np.float32)
    vals = codecs.decode_e2m1(codes) * np.repeat(bs, 16, axis=1)[:, :d]
    return torch.from_numpy(vals.astype(np.float32).reshape(*lead, d)).to(rows.device)


# ------------------------------------------------------------------------------------------ 4-bit activations
_E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def _e2m1_codes(a: torch.Tensor) -> torch.Tensor:
    """Nearest E2M1 magnitude index (ties to the even index, saturating at 6) of non-negative fp32 values."""
    a = a.clamp(max=6.0)
    hi = torch.bucketize(a, _E2M1_VALUES).clamp(max=7)
    lo = (hi - 1).clamp(min=0)
    dlo, dhi = (a - _E2M1_VALUES[lo]).abs(), (_E2M1_VALUES[hi] - a).abs()
    return torch.where((dhi < dlo) | ((dhi == dlo) & ((hi & 1) == 0)), hi, lo)


def quant_act_fp4(x: torch.Tensor, fmt: str):
    """Oracle of the activation quantiser of the W4A4 path (csrc/gemm_fp4.cu): x [T, K] -> (codes uint8 [T, K_pad / 2]
    with element 2 i in the low nibble, block scales uint8 [T, K_pad / block], row scales fp32 [T]); K padded to 256."""
    t, k = x.shape
    block = 32 if fmt == "mxfp4" else 16
    k_pad = (k + 255) // 256 * 256
    xf = torch.zeros((t, k_pad), dtype=torch.float32)
    xf[:, :k] = x.float()
    blk = xf.view(t, k_pad // block, block)
    finite = torch.where(torch.isfinite(blk), blk.abs(), torch.zeros_like(blk))
    bamax = finite.amax(dim=2)
    if fmt == "mxfp4":
        outer = torch.ones(t, dtype=torch.float32)
        bits = bamax.contiguous().view(torch.int32).to(torch.int64) + 0x00200000
        code = (((bits >> 23) & 0xFF) - 2).clamp(0, 254)
        code = torch.where(bamax > 0, code, torch.zeros_like(code))
        scale = torch.where(bamax > 0, torch.ldexp(torch.ones_like(bamax), (code - 127).to(torch.int32)), torch.zeros_like(bamax))
        sf = code.to(torch.uint8)
    else:
        amax = finite.view(t, -1).amax(dim=1)
        outer = torch.where(amax > 0, amax / 2688.0, torch.ones_like(amax)).float()
        want = ((bamax / 6.0) / outer[:, None]).clamp(max=448.0)
        sf = want.to(torch.float8_e4m3fn).view(torch.uint8)
        scale = sf.view(torch.float8_e4m3fn).float() * outer[:, None]
    safe = torch.where(scale > 0, scale, torch.ones_like(scale))
    q = blk / safe.unsqueeze(-1)
    idx = _e2m1_codes(torch.nan_to_num(q.abs(), nan=0.0))
    codes = idx | (((q < 0) & (idx != 0)).to(torch.int64) << 3)
    codes = torch.where((scale > 0).unsqueeze(-1), codes, torch.zeros_like(codes)).view(t, k_pad // 2, 2)
    packed = (codes[..., 0] | (codes[..., 1] << 4)).to(torch.uint8)
    return packed, sf, outer


def dequant_act_fp4(xq: torch.Tensor, xsf: torch.Tensor, outer: torch.Tensor, fmt: str) -> torch.Tensor:
    """fp32 [T, K_pad] of what `quant_act_fp4` (or the kernel) wrote."""
    xq, xsf, outer = xq.cpu(), xsf.cpu(), outer.cpu().float()
    t = xq.shape[0]
    block = 32 if fmt == "mxfp4" else 16
    codes = torch.stack([xq & 0xF, xq >> 4], dim=-1).view(t, -1).long()
    mag = _E2M1_VALUES[codes & 7]
    vals = torch.where((codes & 8) != 0, -mag, mag)
    if fmt == "mxfp4":
        s = torch.ldexp(torch.ones(xsf.shape), xsf.to(torch.int32) - 127)
    else:
        s = xsf.view(torch.float8_e4m3fn).float()
    s = s[:, :vals.shape[1] // block]
    return vals * s.repeat_interleave(block, dim=1) * outer[:, None]

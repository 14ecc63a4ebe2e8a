"""Bit-exact host codecs for the quantised weight and KV-cache encodings.

Everything here is NumPy on the host: it is the compatibility contract used by the GGUF converter,
the checkpoint reader and the numerics oracles; the device kernels are tested against it.

Encodings and rules (reference: crates/sllm-core/src/fp8.rs:36-63,201-275, nvfp4.rs:17-178,
mxfp.rs:11-130, docs/quantization/nvfp4.md:18-31):
  * E4M3FN: round to nearest even, saturate finite values to +-448 (0x7e / 0xfe), NaN -> 0x7f.
  * E4M3FNUZ (MI300 flavour, conversion only): bias 8, no -0, NaN = 0x80, max 240.
  * E2M1 (FP4): values {0, .5, 1, 1.5, 2, 3, 4, 6}; ties go to the code with an even mantissa bit.
  * E8M0: 2^(code - 127); 0 -> 2^-127, 255 = NaN (rejected).
  * FP8 weights: fp32 scale per output row ("outer") or per 128-wide K block ("kblock").
  * NVFP4: 16-element blocks along K, E4M3 block scale, fp32 tensor scale = amax / (448 * 6),
    two codes per byte, low nibble = even index.
  * MXFP4: 32-element blocks along K, E8M0 scale.
"""
from __future__ import annotations

import numpy as np

E4M3_MAX = 448.0
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


# ---------------------------------------------------------------------------------------------- E4M3FN
def _build_e4m3_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 7
        if e == 0xF and m == 7:
            t[b] = np.nan
        elif e == 0:
            t[b] = s * (m / 8.0) * 2.0 ** -6
        else:
            t[b] = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
    return t


E4M3_TABLE = _build_e4m3_table()
_E4M3_POS = E4M3_TABLE[:0x7F].astype(np.float64)  # 0 .. 448, ascending


def decode_e4m3fn(b: np.ndarray) -> np.ndarray:
    return E4M3_TABLE[np.asarray(b, dtype=np.uint8)]


def encode_e4m3fn(x: np.ndarray) -> np.ndarray:
    """float -> E4M3FN byte, RNE, finite values saturate to +-448, NaN -> 0x7f (sign dropped)."""
    xf = np.asarray(x, dtype=np.float32)
    a = np.abs(xf).astype(np.float64)
    nan = np.isnan(xf)
    a = np.where(nan, 0.0, np.minimum(a, E4M3_MAX))
    hi = np.searchsorted(_E4M3_POS, a, side="left")
    hi = np.clip(hi, 0, len(_E4M3_POS) - 1)
    lo = np.clip(hi - 1, 0, len(_E4M3_POS) - 1)
    dlo = np.abs(a - _E4M3_POS[lo])
    dhi = np.abs(_E4M3_POS[hi] - a)
    pick_hi = (dhi < dlo) | ((dhi == dlo) & ((hi & 1) == 0))  # ties -> even code
    code = np.where(pick_hi, hi, lo).astype(np.uint8)
    sign = (np.signbit(xf) & ~nan).astype(np.uint8) << 7
    out = code | sign
    return np.where(nan, np.uint8(0x7F), out).astype(np.uint8)


# ---------------------------------------------------------------------------------------------- E4M3FNUZ
def _build_fnuz_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for b in range(256):
        if b == 0x80:
            t[b] = np.nan
            continue
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 7
        t[b] = s * ((m / 8.0) * 2.0 ** -7 if e == 0 else (1.0 + m / 8.0) * 2.0 ** (e - 8))
    return t


E4M3FNUZ_TABLE = _build_fnuz_table()


def decode_e4m3fnuz(b: np.ndarray) -> np.ndarray:
    return E4M3FNUZ_TABLE[np.asarray(b, dtype=np.uint8)]


def fn_to_fnuz_table() -> np.ndarray:
    """256-entry byte map from E4M3FN codes to the nearest E4M3FNUZ code of the same value (values
    above 240 saturate; NaN -> 0x80; -0 -> +0)."""
    pos = E4M3FNUZ_TABLE[:0x80].astype(np.float64)
    out = np.zeros(256, dtype=np.uint8)
    for b in range(256):
        v = float(E4M3_TABLE[b])
        if np.isnan(v):
            out[b] = 0x80
            continue
        a = min(abs(v), 240.0)
        idx = int(np.argmin(np.abs(pos - a)))
        out[b] = idx | (0x80 if v < 0 and idx != 0 else 0)
    return out


# ---------------------------------------------------------------------------------------------- FP8 weights
def quantize_fp8_outer_rows(w: np.ndarray):
    """[N, K] -> (codes [N, K] uint8, scales [N] fp32); scale = row amax / 448 (1.0 for a zero row)."""
    w = np.asarray(w, dtype=np.float32)
    finite = np.where(np.isfinite(w), np.abs(w), 0.0)
    amax = finite.max(axis=1)
    scale = np.where(amax > 0, amax / np.float32(E4M3_MAX), np.float32(1.0)).astype(np.float32)
    return encode_e4m3fn(w / scale[:, None]), scale


def quantize_fp8_k_blocks(w: np.ndarray, block: int = 128):
    """[N, K] -> (codes [N, K] uint8, scales [N, ceil(K/block)] fp32), one scale per 1 x block tile."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    nb = (k + block - 1) // block
    pad = nb * block - k
    wp = np.pad(w, ((0, 0), (0, pad))) if pad else w
    blk = wp.reshape(n, nb, block)
    finite = np.where(np.isfinite(blk), np.abs(blk), 0.0)
    amax = finite.max(axis=2)
    scale = np.where(amax > 0, amax / np.float32(E4M3_MAX), np.float32(1.0)).astype(np.float32)
    codes = encode_e4m3fn(blk / scale[:, :, None]).reshape(n, nb * block)[:, :k]
    return np.ascontiguousarray(codes), scale


def dequantize_fp8_k_blocks(codes: np.ndarray, scale: np.ndarray, block: int = 128) -> np.ndarray:
    n, k = codes.shape
    s = np.repeat(scale, block, axis=1)[:, :k]
    return decode_e4m3fn(codes) * s


def dequantize_fp8_outer_rows(codes: np.ndarray, scale: np.ndarray) -> np.ndarray:
    return decode_e4m3fn(codes) * scale[:, None]


# ---------------------------------------------------------------------------------------------- E2M1 / NVFP4 / MXFP4
def decode_e2m1(code: np.ndarray) -> np.ndarray:
    c = np.asarray(code, dtype=np.uint8)
    mag = E2M1_VALUES[c & 7]
    return np.where(c & 8, -mag, mag).astype(np.float32)


def encode_e2m1(x: np.ndarray) -> np.ndarray:
    """float -> 4-bit code (sign | 3-bit index); saturate to +-6; ties -> even index; NaN -> 0."""
    xf = np.asarray(x, dtype=np.float32)
    a = np.minimum(np.abs(np.nan_to_num(xf, nan=0.0, posinf=6.0, neginf=6.0)), 6.0).astype(np.float64)
    vals = E2M1_VALUES.astype(np.float64)
    hi = np.clip(np.searchsorted(vals, a, side="left"), 0, 7)
    lo = np.clip(hi - 1, 0, 7)
    dlo, dhi = np.abs(a - vals[lo]), np.abs(vals[hi] - a)
    pick_hi = (dhi < dlo) | ((dhi == dlo) & ((hi & 1) == 0))
    idx = np.where(pick_hi, hi, lo).astype(np.uint8)
    sign = (np.signbit(xf) & ~np.isnan(xf) & (idx != 0)).astype(np.uint8) << 3
    return (idx | sign).astype(np.uint8)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """[..., K] 4-bit codes -> [..., ceil(K/2)] bytes, low nibble = even index."""
    c = np.asarray(codes, dtype=np.uint8)
    if c.shape[-1] % 2:
        c = np.concatenate([c, np.zeros(c.shape[:-1] + (1,), dtype=np.uint8)], axis=-1)
    return (c[..., 0::2] | (c[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray, k: int) -> np.ndarray:
    p = np.asarray(packed, dtype=np.uint8)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = p & 0xF
    out[..., 1::2] = p >> 4
    return out[..., :k]


def quantize_nvfp4(w: np.ndarray, tensor_scale: float | None = None):
    """[N, K] -> (packed [N, ceil(K/2)], block_scales E4M3 [N, ceil(K/16)], tensor_scale fp32).

    tensor_scale = amax / (448 * 6); block scale = (block_amax / 6) / tensor_scale encoded as E4M3;
    a block whose encoded scale is zero stores all-zero codes."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    nb = (k + 15) // 16
    pad = nb * 16 - k
    wp = np.pad(w, ((0, 0), (0, pad))) if pad else w
    blk = wp.reshape(n, nb, 16)
    finite = np.where(np.isfinite(blk), np.abs(blk), 0.0)
    amax = float(finite.max()) if finite.size else 0.0
    ts = np.float32(tensor_scale) if tensor_scale is not None else np.float32(amax / (E4M3_MAX * 6.0) if amax > 0 else 1.0)
    bamax = finite.max(axis=2)
    bs_codes = encode_e4m3fn((bamax / np.float32(6.0)) / ts)
    bs = decode_e4m3fn(bs_codes) * ts
    safe = np.where(bs > 0, bs, np.float32(1.0))
    codes = encode_e2m1(blk / safe[:, :, None])
    codes = np.where((bs > 0)[:, :, None], codes, np.uint8(0)).reshape(n, nb * 16)[:, :k]
    return pack_nibbles(codes), bs_codes.astype(np.uint8), ts


def dequantize_nvfp4(packed: np.ndarray, block_scales: np.ndarray, tensor_scale, k: int) -> np.ndarray:
    codes = unpack_nibbles(packed, k)
    s = np.repeat(decode_e4m3fn(block_scales) * np.float32(tensor_scale), 16, axis=1)[:, :k]
    return decode_e2m1(codes) * s


# ---------------------------------------------------------------------------------------------- GGML super-blocks
# GGUF stores 4-bit tensors as standard GGML blocks (reference: crates/sllm-core/src/gguf_convert.rs:33-143, lossless
# regrouping of its adjacent-pair nibble planes):
#   MXFP4 (type 39): per 32 elements 17 bytes = E8M0 scale, then 16 bytes with byte i = code[i] | code[i + 16] << 4
#   NVFP4 (type 40): per 64 elements 36 bytes = four E4M3 block-16 scales, then per sub-block of 16 elements 8 bytes
#                    with byte i = code[i] | code[i + 8] << 4; the FP32 tensor scale travels as its own tensor
def _to_ggml_halves(codes: np.ndarray, span: int) -> np.ndarray:
    """[..., K] codes -> bytes grouped per `span` elements as (element i | element i + span / 2 << 4)."""
    c = codes.reshape(codes.shape[:-1] + (codes.shape[-1] // span, 2, span // 2))
    return (c[..., 0, :] | (c[..., 1, :] << 4)).astype(np.uint8)          # [..., K / span, span / 2]


def _from_ggml_halves(b: np.ndarray, span: int) -> np.ndarray:
    lo, hi = b & 0xF, b >> 4                                              # [..., blocks, span / 2]
    return np.concatenate([lo, hi], axis=-1).reshape(b.shape[:-2] + (b.shape[-2] * span,)).astype(np.uint8)


def to_ggml_mxfp4(packed: np.ndarray, scales: np.ndarray, k: int) -> bytes:
    """Adjacent-pair codes [N, K/2] + E8M0 scales [N, K/32] -> GGML MXFP4 blocks (K a multiple of 32)."""
    if k % 32:
        raise ValueError("MXFP4 rows must be a multiple of 32 elements")
    q = _to_ggml_halves(unpack_nibbles(packed, k), 32)                    # [N, K/32, 16]
    out = np.concatenate([np.asarray(scales, dtype=np.uint8)[..., None], q], axis=-1)
    return np.ascontiguousarray(out).tobytes()


def from_ggml_mxfp4(raw, n: int, k: int):
    b = np.frombuffer(raw, dtype=np.uint8).reshape(n, k // 32, 17)
    return pack_nibbles(_from_ggml_halves(b[..., 1:], 32)), np.ascontiguousarray(b[..., 0])


def to_ggml_nvfp4(packed: np.ndarray, block_scales: np.ndarray, k: int) -> bytes:
    """Adjacent-pair codes [N, K/2] + E4M3 block-16 scales [N, K/16] -> GGML NVFP4 blocks (K a multiple of 64)."""
    if k % 64:
        raise ValueError("NVFP4 rows must be a multiple of 64 elements")
    n = packed.shape[0]
    q = _to_ggml_halves(unpack_nibbles(packed, k), 16).reshape(n, k // 64, 32)
    sc = np.asarray(block_scales, dtype=np.uint8).reshape(n, k // 64, 4)
    return np.ascontiguousarray(np.concatenate([sc, q], axis=-1)).tobytes()


def from_ggml_nvfp4(raw, n: int, k: int):
    b = np.frombuffer(raw, dtype=np.uint8).reshape(n, k // 64, 36)
    codes = _from_ggml_halves(b[..., 4:].reshape(n, k // 16, 8), 16)
    return pack_nibbles(codes), np.ascontiguousarray(b[..., :4].reshape(n, k // 16))


def decode_e8m0(code: np.ndarray) -> np.ndarray:
    c = np.asarray(code, dtype=np.uint8)
    if np.any(c == 255):
        raise ValueError("E8M0 scale 255 is NaN and is rejected")
    return np.ldexp(np.float64(1.0), c.astype(np.int32) - 127).astype(np.float32)  # code 0 -> 2^-127 (subnormal)


def encode_e8m0_for_amax(amax: np.ndarray, mode: str = "even") -> np.ndarray:
    """Scale code for a block whose largest magnitude is amax.

    'even' (the reference's activation/weight recipe, matmul_kernel.hip.cpp:188-205): round amax at the
    E2M1 mantissa boundary (add a quarter of the mantissa range to the fp32 bits), keep the biased
    exponent, subtract E2M1's maximum exponent 2, clamp to [0, 254]; zero -> 0; non-finite -> 255.
    'floor': exponent of amax minus 2 without the rounding step."""
    a = np.ascontiguousarray(np.asarray(amax, dtype=np.float32))
    bits = a.view(np.uint32).astype(np.uint64)
    if mode == "even":
        bits = bits + 0x00200000
    exp = ((bits & 0x7F800000) >> 23).astype(np.int64) - 2
    code = np.clip(exp, 0, 254)
    code = np.where(a == 0, 0, code)
    code = np.where(np.isfinite(a), code, 255)
    return code.astype(np.uint8)


def quantize_mxfp4(w: np.ndarray, mode: str = "even"):
    """[N, K] -> (packed [N, ceil(K/2)], scales E8M0 [N, ceil(K/32)])."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    nb = (k + 31) // 32
    pad = nb * 32 - k
    wp = np.pad(w, ((0, 0), (0, pad))) if pad else w
    blk = wp.reshape(n, nb, 32)
    finite = np.where(np.isfinite(blk), np.abs(blk), 0.0)
    sc = encode_e8m0_for_amax(finite.max(axis=2), mode)
    s = decode_e8m0(sc)
    codes = encode_e2m1(blk / s[:, :, None]).reshape(n, nb * 32)[:, :k]
    return pack_nibbles(codes), sc


def dequantize_mxfp4(packed: np.ndarray, scales: np.ndarray, k: int) -> np.ndarray:
    codes = unpack_nibbles(packed, k)
    s = np.repeat(decode_e8m0(scales), 32, axis=1)[:, :k]
    return decode_e2m1(codes) * s


def decode_mxfp8(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """MXFP8: E4M3 values with one E8M0 scale per 32 elements."""
    k = codes.shape[-1]
    s = np.repeat(decode_e8m0(scales), 32, axis=-1)[..., :k]
    return decode_e4m3fn(codes) * s


# ---------------------------------------------------------------------------------------------- KV cache encodings
def quantize_kv_fp8(x: np.ndarray, static_scale: float = 0.0):
    """[T, H, D] -> (E4M3 codes, scales [T, H]); scale = amax / 448 per (token, head), Inf saturates."""
    x = np.asarray(x, dtype=np.float32)
    if static_scale > 0:
        scale = np.full(x.shape[:-1], static_scale, dtype=np.float32)
    else:
        finite = np.where(np.isfinite(x), np.abs(x), 0.0)
        amax = finite.max(axis=-1)
        scale = np.where(amax > 0, amax / np.float32(E4M3_MAX), np.float32(1.0)).astype(np.float32)
    return encode_e4m3fn(x / scale[..., None]), scale


def quantize_kv_nvfp4(x: np.ndarray):
    """[T, H, D] -> (packed [T, H, D/2], block scales E4M3 [T, H, D/16], outer fp32 [T, H]);
    outer = amax / (448 * 6) per (token, head); NaN -> 0, Inf saturates."""
    x = np.nan_to_num(np.asarray(x, dtype=np.float32), nan=0.0, posinf=np.float32(3.0e38), neginf=np.float32(-3.0e38))
    t, h, d = x.shape
    nb = (d + 15) // 16
    flat = x.reshape(t * h, d)
    if nb * 16 != d:
        flat = np.pad(flat, ((0, 0), (0, nb * 16 - d)))
    blk = flat.reshape(t * h, nb, 16)
    mag = np.abs(blk)
    amax = mag.max(axis=(1, 2))
    outer = np.where(amax > 0, amax / np.float32(E4M3_MAX * 6.0), np.float32(1.0)).astype(np.float32)
    bs_codes = encode_e4m3fn((mag.max(axis=2) / np.float32(6.0)) / outer[:, None])
    bs = decode_e4m3fn(bs_codes) * outer[:, None]
    safe = np.where(bs > 0, bs, np.float32(1.0))
    codes = encode_e2m1(blk / safe[:, :, None])
    codes = np.where((bs > 0)[:, :, None], codes, np.uint8(0)).reshape(t * h, nb * 16)[:, :d]
    return (pack_nibbles(codes).reshape(t, h, -1), bs_codes.astype(np.uint8).reshape(t, h, -1), outer.reshape(t, h))


def round_bf16(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 (RNE) -> fp32, NaN preserved."""
    xf = np.asarray(x, dtype=np.float32)
    bits = xf.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    out = rounded.view(np.float32)
    return np.where(np.isnan(xf), xf, out)

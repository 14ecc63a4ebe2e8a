"""Tensor-core prefill attention front end (kernel in csrc/prefill_attention.cu).

Used for fresh prompts (every sequence starts at position 0 and its tokens are contiguous rows of the
packed qkv activation) with head_dim 128 and no sliding window; other cases read the paged cache.
"""
from __future__ import annotations

import math

import torch

from . import _lib
from .core import QTensor, _alloc_q, _p, _stream, workspace

MIN_TOKENS = 128
TILE = 128


def usable(q, batch, hd, window, sinks, qkv) -> bool:
    if not q.is_cuda or qkv is None or batch.cu_seqlens is None or sinks is not None or window:
        return False
    if hd != 128 or batch.max_seqlen < MIN_TOKENS or batch.cu_seqlens_host is None:
        return False
    return hasattr(_lib.kernels(), "sllm_prefill_attention")


def build_tiles(cu_seqlens: list, device) -> torch.Tensor:
    """[num_tiles, 4] int32 = (first token row, sequence length, q0, 0); most work first."""
    tiles = []
    for s in range(len(cu_seqlens) - 1):
        t0, n = cu_seqlens[s], cu_seqlens[s + 1] - cu_seqlens[s]
        for q0 in range(0, n, TILE):
            tiles.append((t0, n, q0, 0))
    tiles.sort(key=lambda t: -t[2])
    return torch.tensor(tiles, dtype=torch.int32, device=device)


def prefill_attention(qkv, batch, hq, hkv, hd, *, sm_scale=None, quant_out=False):
    t = qkv.shape[0]
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(hd)
    if batch.prefill_tiles is None:
        batch.prefill_tiles = build_tiles(batch.cu_seqlens_host, qkv.device)
    tiles = batch.prefill_tiles
    wsp = workspace(qkv.device)
    if quant_out:
        oq = _alloc_q(t, hq * hd, qkv.device)
        ob, o8, osc, ld = None, oq.data, oq.scale, t
    else:
        obt = torch.empty((t, hq * hd), dtype=torch.bfloat16, device=qkv.device)
        ob, o8, osc, ld = obt, None, None, 0
    rc = _lib.kernels().sllm_prefill_attention(_p(qkv), t, qkv.stride(0), _p(tiles), tiles.shape[0], hq, hkv, hd, scale,
                                               _p(ob), _p(o8), _p(osc), ld, _p(wsp.status), _stream())
    _lib.check(rc, "prefill_attention")
    return oq if quant_out else obt

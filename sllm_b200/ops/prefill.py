"""Tensor-core prefill attention front end (kernel in csrc/prefill_attention.cu)."""
from __future__ import annotations

import torch

from . import _lib

MIN_TOKENS = 256


def usable(q, batch, hd, window, sinks, qkv) -> bool:
    if not q.is_cuda or qkv is None or batch.cu_seqlens is None or sinks is not None or window:
        return False
    if hd != 128 or batch.max_seqlen < MIN_TOKENS:
        return False
    lib = _lib.kernels()
    return hasattr(lib, "sllm_prefill_attention")


def prefill_attention(qkv, batch, hq, hkv, hd, *, sm_scale=None, quant_out=False):
    raise NotImplementedError

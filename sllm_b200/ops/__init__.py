"""Op layer: hand-written sm_100a kernels for CUDA tensors, PyTorch restatements for CPU tensors."""
from .core import (KVLayer, LinearWeight, QTensor, Workspace, argmax, device_status, elementwise, embedding,
                   gated_act, gemm_raw, linear, paged_attention, quant_fp8, rmsnorm, rope_kv_append, workspace)
from ._lib import KernelError, kernels_available


def attention(q, kv, batch, hq, hkv, hd, *, window=0, quant_out=False, sm_scale=None, sinks=None, qkv=None):
    """Attention for a ForwardBatch.  Fresh long prompts on CUDA take the tensor-core prefill kernel
    (K/V read from the just-computed ``qkv`` activations); everything else reads the paged cache."""
    from . import prefill
    if prefill.usable(q, batch, hd, window, sinks, qkv):
        return prefill.prefill_attention(qkv, batch, hq, hkv, hd, sm_scale=sm_scale, quant_out=quant_out)
    return paged_attention(q, kv, batch.block_table, batch.seq_index, batch.kv_lens, hq, hkv, hd, window=window,
                           sm_scale=sm_scale, max_kv=batch.max_kv, quant_out=quant_out, sinks=sinks)

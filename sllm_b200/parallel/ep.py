"""Expert parallelism: which experts a rank owns and how the expert outputs are combined across ranks.

Activations are replicated across the expert-parallel ranks (they leave the attention all-reduce that way), so
"dispatch" is a local gather of the tokens routed to this rank's experts; "combine" adds the ranks' partial
outputs.  `FusedEP` does the combine in ONE kernel that stores each partial token block into every peer's
receive slot over NVLink and sums in rank order (csrc/moe.cu: moe_combine_allreduce); `NcclEP` is the unfused
baseline (local combine kernel + NCCL all-reduce).  The reference has no expert parallelism
(docs/architecture/runtime.md:554 "no multi-GPU path").
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib, moe as M


class NoEP:
    size, rank = 1, 0

    def expert_range(self, n_experts: int):
        return 0, n_experts

    def combine(self, yp, perm_dst, residual):
        return M.combine(yp, perm_dst, residual)


class NcclEP(NoEP):
    impl = "nccl"

    def __init__(self, size: int, rank: int, device, group=None):
        self.size, self.rank, self.device, self.group = size, rank, torch.device(device), group

    def expert_range(self, n_experts: int):
        if n_experts % self.size:
            raise ValueError("experts must divide evenly across expert-parallel ranks")
        per = n_experts // self.size
        return self.rank * per, (self.rank + 1) * per

    def combine(self, yp, perm_dst, residual):
        # the residual is added once, after the reduction
        part = M.combine(yp, perm_dst, None)
        if self.size > 1:
            part = part.float() if not part.is_cuda else part
            dist.all_reduce(part, group=self.group)
        if residual is not None:
            part = (part.float() + residual.float()).to(residual.dtype)
        return part

    def close(self):
        pass


class FusedEP(NcclEP):
    impl = "fused"

    def __init__(self, size: int, rank: int, device, max_tokens: int, d_model: int, group=None, rows_per_block: int = 4):
        super().__init__(size, rank, device, group)
        from .symm import SymmetricRegion
        self.max_tokens, self.d = max_tokens, d_model
        self.rows_per_block = rows_per_block
        self.cap = max_tokens * d_model
        self.max_blocks = (max_tokens + rows_per_block - 1) // rows_per_block
        recv_bytes = 2 * size * self.cap * 2
        flag_bytes = size * self.max_blocks * 4
        self.region = SymmetricRegion(recv_bytes + flag_bytes + 4096, size, rank, group)
        self.off_recv = self.region.carve(recv_bytes)
        self.off_flags = self.region.carve(flag_bytes)
        self._recv = self.region.peer_array(self.off_recv)
        self._flags = self.region.peer_array(self.off_flags)
        self.epoch = torch.zeros(self.max_blocks, dtype=torch.int32, device=device)

    def combine(self, yp, perm_dst, residual):
        t, k = perm_dst.shape
        if not yp.is_cuda or t > self.max_tokens:
            return super().combine(yp, perm_dst, residual)
        from ..ops.core import _p, _stream, workspace
        y = torch.empty((t, self.d), dtype=torch.bfloat16, device=yp.device)
        rc = M._k().sllm_moe_combine_allreduce(
            C.cast(self._recv, C.c_void_p), C.cast(self._flags, C.c_void_p), self.size, self.rank, _p(yp), _p(perm_dst), k,
            _p(residual), _p(y), t, self.d, self.rows_per_block, self.cap, self.max_blocks, _p(self.epoch),
            _p(workspace(yp.device).status), _stream())
        _lib.check(rc, "moe_combine_allreduce")
        return y

    def close(self):
        if self.region is not None:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            self.region.close()
            self.region = None

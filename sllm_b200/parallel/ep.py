"""Expert parallelism: which experts a rank owns and how the expert outputs are combined across ranks.

Activations are replicated across the expert-parallel ranks (they leave the attention all-reduce that way), so
"dispatch" needs no transfer: a rank gathers the tokens routed to its experts locally.  "Combine" is where bytes
move.  `FusedEP.experts_combine` runs the token-owner path (csrc/moe.cu, "owner combine"): the down-projection GEMM
of every rank stores each routed row, route weight applied, straight into the receive slot of the token's OWNER over
NVLink (scatter epilogue of the grouped W4 GEMM); owners sum their tokens' top-k slots in slot order, add the
residual and store the finished rows into every rank's gather buffer.  A rank sends the rows its experts produced
plus its own tokens' results, instead of a full partial of every token to every peer (`FusedEP.combine`, the earlier
all-reduce form, kept for callers that hold permuted expert outputs already).  `NcclEP` is the unfused baseline
(local combine kernel + NCCL all-reduce).  The reference has no expert parallelism
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

    def experts_combine(self, x, idx, rw, gate_up, down, act: str, e_lo: int, e_hi: int, residual):
        """Routed experts of this rank on `x` and the sum over all ranks (+ residual): the MoE block after routing."""
        yp, perm_dst = M.experts_forward(x, idx, rw, gate_up, down, act, e_lo, e_hi)
        return self.combine(yp, perm_dst, residual)


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
        # token-owner path: receive slots [2][tokens per rank x top-k x d], gather buffer [2][tokens x d], two flag rows
        self.top_k_cap = 8
        self.tpr_cap = (max_tokens + size - 1) // size
        self.slot_cap = self.tpr_cap * self.top_k_cap * d_model
        slot_bytes, gath_bytes, oflag_bytes = 2 * self.slot_cap * 2, 2 * self.cap * 2, 2 * size * 4
        self.owner_region = SymmetricRegion(slot_bytes + gath_bytes + oflag_bytes + 4096, size, rank, group)
        self._oslots = self.owner_region.peer_array(self.owner_region.carve(slot_bytes))
        self._ogath = self.owner_region.peer_array(self.owner_region.carve(gath_bytes))
        self._oflags = self.owner_region.peer_array(self.owner_region.carve(oflag_bytes))
        self.owner_epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.owner_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.owner_path = True

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

    def experts_combine(self, x, idx, rw, gate_up, down, act: str, e_lo: int, e_hi: int, residual):
        t, k = idx.shape
        if not (self.owner_path and x.is_cuda and t <= self.max_tokens and k <= self.top_k_cap and down.n == self.d):
            if x.is_cuda:
                _lib.note_fallback("ep_owner_combine:outside_limits")
            return super().experts_combine(x, idx, rw, gate_up, down, act, e_lo, e_hi, residual)
        from ..ops import core
        from ..ops.core import _p, _stream, workspace
        from ..ops.w4 import linear_w4
        lib = M._k()
        P, I, L = C.c_void_p, C.c_int, C.c_longlong
        tok_off, perm_src, perm_dst, perm_w = M.permute(idx, rw, e_lo, e_hi)
        tpr = (t + self.size - 1) // self.size
        row_ptr = torch.empty(t * k, dtype=torch.int64, device=x.device)
        peers = (C.cast(self._oslots, P), C.cast(self._ogath, P), C.cast(self._oflags, P), self.size, self.rank,
                 self.slot_cap, self.cap)
        rc = lib.sllm_moe_owner_plan(*peers, _p(perm_dst), t, k, self.d, tpr, _p(self.owner_epoch), _p(row_ptr), _stream())
        _lib.check(rc, "moe_owner_plan")
        # the down projection stores every routed row (route weight applied) into its owner's slot, on whatever GPU
        M.expert_mlp(x, tok_off, perm_src, perm_w, gate_up, down, act, row_ptr=row_ptr)
        y = torch.empty((t, self.d), dtype=torch.bfloat16, device=x.device)
        rc = lib.sllm_moe_owner_combine(*peers, k, _p(residual), _p(y), t, self.d, tpr, self.rows_per_block,
                                        _p(self.owner_epoch), _p(self.owner_counter), _p(workspace(x.device).status), _stream())
        _lib.check(rc, "moe_owner_combine")
        return y

    def close(self):
        if self.region is not None:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            self.region.close()
            self.owner_region.close()
            self.region = None

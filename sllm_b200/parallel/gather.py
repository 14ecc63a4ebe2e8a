"""All-gather fused into a column-parallel GEMM over symmetric peer memory.

Every rank holds a K shard X_r [rows, k / world] of the activations (the layout a reduce-scatter over the
feature axis leaves behind) and its own rows W [n_local, k] of a column-parallel weight.  `GatherGemm.linear`
publishes the shard (one small kernel: copy into the rank's symmetric buffer, raise a flag on every rank) and runs
the tcgen05 GEMM whose TMA producer pulls the peers' shards straight out of their memory, own shard first, each
behind a bounded wait on its owner's flag: the MMAs of the shards already there overlap the NVLink transfer of the
rest.  Plain TMA loads only, no cluster multicast.  `NcclGatherGemm` is the unfused comparator
(all_gather_into_tensor, then the same GEMM on local memory).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _lib
from ..ops.core import LinearWeight, _gemm_plan, _p, _stream, workspace

_lib.EXTRA_KERNEL_SIGNATURES.update({
    "sllm_gather_build_maps": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "sllm_gather_publish": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p,
                                       C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "sllm_gemm_allgather": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                       C.c_int, C.c_int, C.c_void_p, C.c_longlong, C.c_void_p, C.c_int, C.c_void_p,
                                       C.c_void_p, C.c_void_p]),
})


class GatherDesc(C.Structure):
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("maps", C.c_void_p), ("flags", C.c_void_p), ("epoch", C.c_void_p)]


class NcclGatherGemm:
    """Unfused comparator: NCCL all-gather of the shards, then the GEMM."""
    impl = "nccl"

    def __init__(self, size: int, rank: int, device, group=None):
        self.size, self.rank, self.device, self.group = size, rank, torch.device(device), group

    def linear(self, x_shard: torch.Tensor, w: LinearWeight, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        rows, ks = x_shard.shape
        flat = torch.empty((self.size * rows, ks), dtype=x_shard.dtype, device=x_shard.device)
        dist.all_gather_into_tensor(flat, x_shard.contiguous(), group=self.group)
        x = flat.view(self.size, rows, ks).permute(1, 0, 2).reshape(rows, self.size * ks).contiguous()
        return ops.linear(x, w, residual)

    def close(self) -> None:
        pass


class GatherGemm(NcclGatherGemm):
    impl = "fused"

    def __init__(self, size: int, rank: int, device, max_rows: int, k: int, group=None):
        super().__init__(size, rank, device, group)
        from .symm import SymmetricRegion
        from .tp import check_comm_abi
        check_comm_abi()
        if k % (64 * size):
            raise ValueError("k must be a multiple of 64 * world (whole 128-byte K blocks per rank)")
        self.max_rows = (max_rows + 127) // 128 * 128 if max_rows > 64 else (16 if max_rows <= 16 else 32 if max_rows <= 32 else 64)
        self.k, self.ks = k, k // size
        buf_bytes = self.max_rows * self.ks * 2
        self.region = SymmetricRegion(2 * buf_bytes + 4096, size, rank, group)
        self.off_buf = [self.region.carve(buf_bytes, 1024), self.region.carve(buf_bytes, 1024)]
        self.off_flags = self.region.carve(64)
        lib = _lib.kernels()
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.maps = torch.zeros(4 * 2 * size * 128, dtype=torch.uint8, device=self.device)
        assert self.maps.data_ptr() % 64 == 0
        bufs = (C.c_void_p * (2 * size))()
        for r in range(size):
            for par in range(2):
                bufs[r * 2 + par] = self.region.ptrs[r] + self.off_buf[par]
        _lib.check(lib.sllm_gather_build_maps(self.maps.data_ptr(), bufs, size, self.max_rows, self.ks), "gather_build_maps")
        _lib.LAUNCH_COUNT[0] -= 1
        self._flags_on_peers = self.region.peer_array(self.off_flags)
        self.desc = GatherDesc(size, rank, self.maps.data_ptr(), self.region.ptrs[rank] + self.off_flags,
                               self.epoch.data_ptr())
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def linear(self, x_shard: torch.Tensor, w: LinearWeight, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        rows, ks = x_shard.shape
        if (w.kind != "dense" or w.w.dtype != torch.bfloat16 or x_shard.dtype != torch.bfloat16 or ks != self.ks
                or w.w.shape[1] != self.k or rows > self.max_rows or not x_shard.is_cuda):
            return super().linear(x_shard, w, residual)
        lib = _lib.kernels()
        n = w.w.shape[0]
        local = self.region.ptrs[self.rank]
        rc = lib.sllm_gather_publish(_p(x_shard), rows, ks, x_shard.stride(0), local + self.off_buf[0],
                                     local + self.off_buf[1], self.max_rows, self.epoch.data_ptr(), self._flags_on_peers,
                                     self.size, self.rank, _stream())
        _lib.check(rc, "gather_publish")
        swap, bn, splits, stages = _gemm_plan(rows, n, self.k // 64)
        if not swap:
            bn = 128
            splits = 1
        y = torch.empty((rows, n), dtype=torch.bfloat16, device=x_shard.device)
        wsp = workspace(x_shard.device)
        rc = lib.sllm_gemm_allgather(_p(w.w), _p(y), _p(residual), n, rows, self.k, y.stride(0), bn, splits, stages,
                                     _p(wsp.ws), wsp.ws.numel(), _p(wsp.counters), wsp.counters.numel(), _p(wsp.status),
                                     _stream(), C.addressof(self.desc))
        _lib.check(rc, "gemm_allgather")
        return y

    def close(self) -> None:
        if self.region is not None:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            self.region.close()
            self.region = None

"""Symmetric peer memory: one same-sized device region per rank, mapped into every rank.

torch.distributed (NCCL or gloo) is used only to exchange the 64-byte IPC handles; the kernels then
address peers directly through the pointer table.  Regions are carved into named slices so several
users (fused GEMM receive buffers, flags, small all-gathers) share one allocation.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib

_lib.EXTRA_KERNEL_SIGNATURES.update({
    "sllm_symm_alloc": (C.c_int, [C.c_longlong, C.POINTER(C.c_void_p), C.c_char_p]),
    "sllm_symm_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "sllm_symm_close": (C.c_int, [C.c_void_p]),
    "sllm_symm_free": (C.c_int, [C.c_void_p]),
    "sllm_allgather_small": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_longlong, C.c_longlong, C.c_int, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_void_p, C.c_void_p]),
    "sllm_argmax_merge": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
})


class SymmetricRegion:
    def __init__(self, nbytes: int, world: int, rank: int, group=None):
        lib = _lib.kernels()
        self.world, self.rank, self.nbytes = world, rank, nbytes
        self.local = C.c_void_p()
        handle = C.create_string_buffer(64)
        _lib.check(lib.sllm_symm_alloc(nbytes, C.byref(self.local), handle), "symm_alloc")
        _lib.LAUNCH_COUNT[0] -= 1
        handles = [None] * world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.ptrs = []
        for r in range(world):
            if r == rank:
                self.ptrs.append(self.local.value)
            else:
                p = C.c_void_p()
                _lib.check(lib.sllm_symm_open(handles[r], C.byref(p)), "symm_open")
                _lib.LAUNCH_COUNT[0] -= 1
                self.ptrs.append(p.value)
        self._cursor = 0
        dist.barrier(group=group)

    def carve(self, nbytes: int, align: int = 256) -> int:
        """Reserve a slice (same offset on every rank); returns the byte offset."""
        off = (self._cursor + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError("symmetric region exhausted")
        self._cursor = off + nbytes
        return off

    def peer_array(self, offset: int = 0):
        arr = (C.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.ptrs[r] + offset
        return arr

    def close(self):
        lib = _lib.kernels()
        for r, p in enumerate(self.ptrs):
            if r != self.rank and p:
                lib.sllm_symm_close(C.c_void_p(p))
        if dist.is_initialized():
            dist.barrier()  # nobody frees a region a peer still has mapped
        if self.local:
            lib.sllm_symm_free(self.local)
            self.local = C.c_void_p()
        self.ptrs = []

"""Tensor-parallel context: how row-parallel projections, logits and argmax cross ranks.

Two implementations with one interface:
  * ``fused``: the row-parallel GEMM and its all-reduce are ONE kernel (csrc/gemm_tcgen05.cu, kComm):
    each finished tile is pushed to the peers' receive buffers over NVLink and summed in rank order.
    Vocabulary-shard argmax records cross ranks through a one-shot peer all-gather kernel.
  * ``nccl``: the unfused comparator - local GEMM, ``dist.all_reduce``, residual add, and
    ``dist.all_gather`` for logits / argmax records.
The reference has no tensor parallelism (docs/architecture/runtime.md:459-461).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _lib
from ..ops.core import LinearWeight, QTensor, _gemm_plan, _p, _stream, workspace

_lib.EXTRA_KERNEL_SIGNATURES["sllm_gemm_allreduce"] = (
    C.c_int, [C.c_void_p] * 6 + [C.c_int] * 11 + [C.c_void_p, C.c_longlong, C.c_void_p, C.c_int, C.c_void_p,
                                                   C.c_void_p, C.c_void_p])


class CommDesc(C.Structure):
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("cap_elems", C.c_longlong), ("max_tiles", C.c_int),
                ("reserved", C.c_int), ("recv", C.c_void_p * 8), ("flags", C.c_void_p * 8), ("epoch", C.c_void_p)]


_abi_ok = False


def check_comm_abi() -> None:
    """Compares the ctypes mirrors of the communicator descriptors with the layout the library was compiled with
    (a silent field-order drift would hand peer pointers to the wrong slots)."""
    global _abi_ok
    if _abi_ok:
        return
    from .gather import GatherDesc
    _lib.EXTRA_KERNEL_SIGNATURES.setdefault("sllm_comm_abi", (C.c_int, [C.POINTER(C.c_int), C.c_int]))
    buf = (C.c_int * 16)()
    n = _lib.kernels().sllm_comm_abi(buf, 16)
    mine = [C.sizeof(CommDesc), CommDesc.recv.offset, CommDesc.flags.offset, CommDesc.epoch.offset,
            C.sizeof(GatherDesc), GatherDesc.maps.offset, GatherDesc.flags.offset, GatherDesc.epoch.offset]
    if n != len(mine) or list(buf[:n]) != mine:
        raise _lib.KernelError(f"communicator descriptor layout mismatch: library {list(buf[:n])}, bindings {mine}")
    _abi_ok = True


class NcclTP:
    """Unfused baseline: library collectives between kernels."""
    impl = "nccl"

    def __init__(self, size: int, rank: int, device, group=None):
        self.size, self.rank, self.device, self.group = size, rank, device, group

    def close(self) -> None:
        pass

    def row_linear(self, x, w: LinearWeight, residual):
        y = ops.linear(x, w)
        dist.all_reduce(y, group=self.group)
        if residual is not None:
            y = ops.elementwise("add", y, residual) if y.is_cuda else y + residual
        return y

    def gather_logits(self, logits: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(logits) for _ in range(self.size)]
        dist.all_gather(parts, logits.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def argmax(self, logits: torch.Tensor, vocab_offset: int) -> torch.Tensor:
        idx, val = ops.argmax(logits, vocab_offset, with_values=True)
        vals = [torch.empty_like(val) for _ in range(self.size)]
        idxs = [torch.empty_like(idx) for _ in range(self.size)]
        dist.all_gather(vals, val, group=self.group)
        dist.all_gather(idxs, idx, group=self.group)
        v, i = torch.stack(vals), torch.stack(idxs)
        return merge_argmax(v, i)


def merge_argmax(vals: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """[world, rows] records -> best index per row (max value, ties lowest index, -1 if any shard saw NaN)."""
    if vals.is_cuda:
        world, rows = vals.shape
        out = torch.empty(rows, dtype=torch.int32, device=vals.device)
        rc = _lib.kernels().sllm_argmax_merge(_p(vals.contiguous()), _p(idx.contiguous()), _p(out), rows, world,
                                              _stream())
        _lib.check(rc, "argmax_merge")
        return out
    best = vals.max(dim=0).values
    cand = torch.where(vals == best.unsqueeze(0), idx, torch.full_like(idx, 2**31 - 1))
    out = cand.min(dim=0).values
    return torch.where((idx < 0).any(dim=0), torch.full_like(out, -1), out)


class FusedTP(NcclTP):
    """Fused compute+collective kernels over symmetric peer memory."""
    impl = "fused"

    def __init__(self, size: int, rank: int, device, max_tokens: int, d_model: int, group=None,
                 max_rows_small: int = 1024):
        super().__init__(size, rank, device, group)
        check_comm_abi()
        from .symm import SymmetricRegion
        self.max_tokens = max_tokens
        self._d_model = d_model
        self._row_reduce = None
        # receive buffers: [2 parities][world][cap] bf16; cap covers a padded [tokens, d_model] tile grid
        pad_tokens = 16 if max_tokens <= 16 else 32 if max_tokens <= 32 else 64 if max_tokens <= 64 else \
            (max_tokens + 127) // 128 * 128
        n_pad = (d_model + 127) // 128 * 128
        self.cap_elems = pad_tokens * n_pad
        self.max_tiles = max(n_pad // 128, (pad_tokens + 127) // 128 * (n_pad // 16))
        recv_bytes = 2 * size * self.cap_elems * 2
        flag_bytes = self.max_tiles * 8 * size * 4   # 8 cluster slices per tile
        small_slot = max_rows_small * 8
        small_bytes = 2 * size * small_slot
        # the fused decode path sums whole 128-row tiles of up to 32 token rows: its own receive buffers, flags and
        # epochs (one slot per tile), so that its slot numbering never meets the per-GEMM kernel's in one region
        self.fd_cap_elems = 32 * n_pad
        self.fd_max_tiles = n_pad // 128
        fd_recv_bytes = 2 * size * self.fd_cap_elems * 2
        fd_flag_bytes = self.fd_max_tiles * size * 4
        total = recv_bytes + flag_bytes + small_bytes + fd_recv_bytes + fd_flag_bytes + 8192
        self.region = SymmetricRegion(total, size, rank, group)
        self.off_recv = self.region.carve(recv_bytes)
        self.off_flags = self.region.carve(flag_bytes)
        self.off_small = self.region.carve(small_bytes)
        self.off_small_flags = self.region.carve(64)
        self.small_slot = small_slot
        self.epoch = torch.zeros(self.max_tiles * 8 + 8, dtype=torch.int32, device=device)
        self.small_epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.desc = CommDesc()
        self.desc.world, self.desc.rank = size, rank
        self.desc.cap_elems, self.desc.max_tiles = self.cap_elems, self.max_tiles
        recv = self.region.peer_array(self.off_recv)
        flags = self.region.peer_array(self.off_flags)
        for r in range(size):
            self.desc.recv[r] = recv[r]
            self.desc.flags[r] = flags[r]
        self.desc.epoch = self.epoch.data_ptr()
        off_fd_recv = self.region.carve(fd_recv_bytes)
        off_fd_flags = self.region.carve(fd_flag_bytes)
        self.fd_epoch = torch.zeros(self.fd_max_tiles + 8, dtype=torch.int32, device=device)
        self.desc_fd = CommDesc()
        self.desc_fd.world, self.desc_fd.rank = size, rank
        self.desc_fd.cap_elems, self.desc_fd.max_tiles = self.fd_cap_elems, self.fd_max_tiles
        fd_recv, fd_flags = self.region.peer_array(off_fd_recv), self.region.peer_array(off_fd_flags)
        for r in range(size):
            self.desc_fd.recv[r] = fd_recv[r]
            self.desc_fd.flags[r] = fd_flags[r]
        self.desc_fd.epoch = self.fd_epoch.data_ptr()
        self._small_bases = self.region.peer_array(0)
        self._small_src = torch.zeros(small_slot, dtype=torch.uint8, device=device)
        self._small_dst = torch.zeros(size * small_slot, dtype=torch.uint8, device=device)

    def close(self) -> None:
        """Unmaps the peers' regions, then frees the local one (all ranks must call this together)."""
        if self._row_reduce is not None:
            self._row_reduce.close()
            self._row_reduce = None
        if self.region is not None:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            self.region.close()
            self.region = None

    def _reduce_rows(self, part: torch.Tensor, residual):
        """All-reduce of [m, n] partial rows (+ residual) in one kernel over peer memory: the expert-parallel
        combine kernel with the identity permutation."""
        if self._row_reduce is None:
            from .ep import FusedEP
            self._row_reduce = FusedEP(self.size, self.rank, self.device, self.max_tokens, self._d_model, self.group)
            self._ident = torch.arange(self.max_tokens, dtype=torch.int32, device=self.device).view(-1, 1)
        return self._row_reduce.combine(part, self._ident[:part.shape[0]], residual)

    def row_linear(self, x, w: LinearWeight, residual):
        xd = x.data if isinstance(x, QTensor) or hasattr(x, "sf") else x      # QTensor, 4-bit activations, or a matrix
        m, n = xd.shape[0], w.out_features
        if not xd.is_cuda or m > self.max_tokens:
            if xd.is_cuda:
                _lib.note_fallback("tp_row_linear_nccl:rows_above_fused_limit")
            return super().row_linear(x, w, residual)
        if w.kind == "w4":
            # 4-bit weights: W4A16 GEMM, then the fused peer-memory reduction
            part = ops.linear(x, w)
            if n != self._d_model:
                _lib.note_fallback("tp_row_linear_nccl:w4_width")
                return super().row_linear(x, w, residual)
            return self._reduce_rows(part, residual)
        lib = _lib.kernels()
        fp8 = w.kind == "fp8"
        if fp8 and not isinstance(x, QTensor):
            x = ops.quant_fp8(x)
        k_blocks = (w.in_features + 127) // 128 if fp8 else (w.in_features + 63) // 64
        swap, bn, splits, stages = _gemm_plan(m, n, k_blocks)
        y = torch.empty((m, n), dtype=torch.bfloat16, device=xd.device)
        wsp = workspace(xd.device)
        if swap:
            a, b = w.w, (x.data if fp8 else x)
            sa, sb = (w.scale_t, x.scale) if fp8 else (None, None)
        else:
            a, b = (x.data if fp8 else x), w.w
            sa, sb = (x.scale, w.scale_t) if fp8 else (None, None)
        rc = lib.sllm_gemm_allreduce(
            _p(a), _p(b), _p(y), _p(sa), _p(sb), _p(residual), a.shape[0], b.shape[0], a.shape[1], int(fp8),
            int(swap), y.stride(0), sa.stride(0) if fp8 else 0, sb.stride(0) if fp8 else 0, bn, splits, stages,
            _p(wsp.ws), wsp.ws.numel(), _p(wsp.counters), wsp.counters.numel(), _p(wsp.status), _stream(),
            C.cast(C.pointer(self.desc), C.c_void_p))
        _lib.check(rc, "gemm_allreduce")
        return y

    def argmax(self, logits: torch.Tensor, vocab_offset: int) -> torch.Tensor:
        rows = logits.shape[0]
        if not logits.is_cuda or rows * 8 > self.small_slot:
            return super().argmax(logits, vocab_offset)
        idx, val = ops.argmax(logits, vocab_offset, with_values=True)
        src = self._small_src
        src[:rows * 4].view(torch.float32).copy_(val)
        src[rows * 4:rows * 8].view(torch.int32).copy_(idx)
        slot = rows * 8
        rc = _lib.kernels().sllm_allgather_small(
            C.cast(self._small_bases, C.c_void_p), self.size, self.rank, self.off_small, self.off_small_flags, slot,
            _p(src),
            _p(self._small_dst), _p(self.small_epoch), _p(workspace(logits.device).status), _stream())
        _lib.check(rc, "allgather_small")
        rec = self._small_dst[:self.size * slot].view(self.size, slot)
        vals = rec[:, :rows * 4].contiguous().view(torch.float32).view(self.size, rows)
        idxs = rec[:, rows * 4:].contiguous().view(torch.int32).view(self.size, rows)
        return merge_argmax(vals, idxs)


def make_tp(size: int, rank: int, device, impl: str = "fused", max_tokens: int = 128, d_model: int = 4096,
            group=None):
    if size == 1:
        return None
    if torch.device(device).type == "cuda":
        # the kernel after decode attention is a GEMM fused with a collective here: measured 10 % slower at two GPUs
        # when its CTAs become resident while the attention grid still drains
        _lib.EXTRA_KERNEL_SIGNATURES.setdefault("sllm_attention_set_early_trigger", (None, [C.c_int]))
        _lib.kernels().sllm_attention_set_early_trigger(0)
    if impl == "fused":
        return FusedTP(size, rank, device, max_tokens, d_model, group)
    return NcclTP(size, rank, device, group)

"""Paged KV-cache manager: device page tensors + the native page pool.

Layout per layer (K and V alike): values ``[num_pages, kv_heads, page, head_dim]`` and, for dynamic
FP8, fp32 scales ``[num_pages, kv_heads, page]`` (one scale per token and head, ``amax / 448``).  The
byte offset of (sequence token t, head h, channel c) inside a sequence's page list is
``page_list[t // page] * page_bytes + ((h * page) + t % page) * head_dim + c``: block-16 paging as in
the reference's layout oracle (tests/reference/oracles.py:209-239, tests/fixtures/kv_layout.json), but
head-major inside a page, so that the 16 tokens of one head are one contiguous 2 KB run in HBM - the
unit one attention CTA fetches with a single TMA box (token-major pages gave 128-byte pieces at a 1 KB
stride and held the decode attention kernel near half of the DRAM bandwidth).

Sequences are handles into the native pool (csrc/host/page_pool.cpp): reserve -> run step -> commit
gives the reference's transactional length publication (docs/architecture/runtime.md:145-149); fork
shares full pages and copies the tail page (its read-only page sharing + COW tail, :323-331).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from ..models.config import ModelConfig
from ..ops import _lib
from ..ops.core import KVLayer


class OutOfPages(RuntimeError):
    pass


def paged_kv_offset(page_list, token: int, head: int, channel: int, page_size: int, kv_heads: int, head_dim: int,
                    elem_bytes: int = 1) -> int:
    """Byte offset of one element inside the value plane of a layer."""
    page = page_list[token // page_size]
    return ((page * kv_heads + head) * page_size + token % page_size) * head_dim * elem_bytes + channel * elem_bytes


class PagePool:
    """Thin wrapper over the native ref-counted pool."""

    def __init__(self, num_pages: int, page_size: int = 16):
        self._lib = _lib.host()
        self._lib.sllm_kv_seq_length.restype = C.c_longlong
        self._lib.sllm_kv_seq_reserve.argtypes = [C.c_int, C.c_int, C.c_longlong]
        self._lib.sllm_kv_seq_commit.argtypes = [C.c_int, C.c_int, C.c_longlong]
        self._lib.sllm_kv_seq_truncate.argtypes = [C.c_int, C.c_int, C.c_longlong]
        self._lib.sllm_kv_seq_fork.argtypes = [C.c_int, C.c_int, C.c_longlong, C.c_void_p]
        self.num_pages = num_pages
        self.page_size = page_size
        self.h = self._lib.sllm_kv_pool_create(num_pages, page_size)
        if self.h <= 0:
            raise ValueError("invalid page pool size")

    def close(self) -> None:
        if self.h > 0:
            self._lib.sllm_kv_pool_destroy(self.h)
            self.h = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def stats(self) -> dict:
        out = (C.c_longlong * 4)()
        self._lib.sllm_kv_pool_stats(self.h, out)
        return {"pages": out[0], "free": out[1], "high_water": out[2], "sequences": out[3]}

    def new_seq(self) -> int:
        return self._lib.sllm_kv_seq_new(self.h)

    def free_seq(self, seq: int) -> None:
        self._lib.sllm_kv_seq_free(self.h, seq)

    def reserve(self, seq: int, new_len: int) -> None:
        rc = self._lib.sllm_kv_seq_reserve(self.h, seq, new_len)
        if rc == 3:
            raise OutOfPages(f"no free KV pages for {new_len} tokens")
        if rc:
            raise ValueError(f"kv reserve failed ({rc})")

    def commit(self, seq: int, new_len: int) -> None:
        rc = self._lib.sllm_kv_seq_commit(self.h, seq, new_len)
        if rc:
            raise ValueError(f"kv commit failed ({rc})")

    def truncate(self, seq: int, length: int) -> None:
        rc = self._lib.sllm_kv_seq_truncate(self.h, seq, length)
        if rc:
            raise ValueError(f"kv truncate failed ({rc})")

    def length(self, seq: int) -> int:
        return int(self._lib.sllm_kv_seq_length(self.h, seq))

    def pages(self, seq: int) -> list:
        cap = 1 << 16
        buf = (C.c_int * cap)()
        n = self._lib.sllm_kv_seq_pages(self.h, seq, buf, cap)
        if n < 0:
            raise KeyError(seq)
        return list(buf[:n])

    def fork(self, seq: int, prefix_len: int):
        pair = (C.c_int * 2)()
        child = self._lib.sllm_kv_seq_fork(self.h, seq, prefix_len, pair)
        if child == -3:
            raise OutOfPages("no free page for the forked tail")
        if child < 0:
            raise ValueError(f"kv fork failed ({-child})")
        return child, (pair[0], pair[1])

    def make_tail_private(self, seq: int):
        pair = (C.c_int * 2)()
        rc = self._lib.sllm_kv_seq_make_tail_private(self.h, seq, pair)
        if rc == -3:
            raise OutOfPages("no free page for a private tail")
        if rc < 0:
            raise ValueError(f"make_tail_private failed ({-rc})")
        return (pair[0], pair[1]) if rc == 1 else None

    def refcount(self, page: int) -> int:
        return self._lib.sllm_kv_page_refcount(self.h, page)

    def inject_alloc_failure(self, after_calls: int) -> None:
        self._lib.sllm_kv_pool_inject_alloc_failure(self.h, after_calls)

    def fill_block_table(self, seqs: list, table: torch.Tensor) -> None:
        """table: int32 CPU tensor [>= len(seqs), max_blocks], contiguous."""
        arr = (C.c_int * len(seqs))(*seqs)
        rc = self._lib.sllm_kv_fill_block_table(self.h, arr, len(seqs), C.c_void_p(table.data_ptr()), table.shape[1])
        if rc:
            raise ValueError(f"block table export failed ({rc})")


@dataclass
class KVSpec:
    n_layers: int
    kv_heads: int
    head_dim: int
    page_size: int
    fmt: str  # fp32 | bf16 | fp8 | fp8-static


class PagedKVCache:
    """Device pages for every layer + the pool.  ``layer(i)`` gives the tensors an op needs."""

    def __init__(self, cfg: ModelConfig, num_pages: int, device: torch.device, kv_heads: Optional[int] = None,
                 k_static: float = 0.0, v_static: float = 0.0, static_scales: Optional[list] = None):
        """``static_scales``: [(k, v)] decode scales per layer for the `fp8-static` format (a quantised checkpoint
        binds one pair per layer: reference crates/sllm-core/src/quantized_model.rs:80-95); otherwise k_static /
        v_static apply to every layer."""
        hkv = kv_heads if kv_heads is not None else cfg.n_kv_heads
        self.spec = KVSpec(cfg.n_layers, hkv, cfg.head_dim, cfg.page_size, cfg.kv_format)
        self.device = device
        self.pool = PagePool(num_pages, cfg.page_size)
        fmt = cfg.kv_format
        if fmt not in ("fp32", "bf16", "fp16", "fp8", "fp8-static", "nvfp4"):
            raise ValueError(f"unknown KV-cache format {fmt!r}")
        self.fp8 = fmt in ("fp8", "fp8-static")
        self.nvfp4 = fmt == "nvfp4"
        if self.nvfp4 and cfg.head_dim % 64:
            raise ValueError("NVFP4 KV rows need a head width that is a multiple of 64")
        vdtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}.get(fmt, torch.uint8)
        # an NVFP4 row holds head_dim / 2 code bytes and head_dim / 16 block-scale bytes (9 bits per value with the
        # fp32 outer scale of the row in the scale plane)
        row = cfg.head_dim // 2 + cfg.head_dim // 16 if self.nvfp4 else cfg.head_dim
        shape = (cfg.n_layers, 2, num_pages, hkv, cfg.page_size, row)
        self.values = torch.zeros(shape, dtype=vdtype, device=device)
        self.scales = None
        if fmt in ("fp8", "nvfp4"):
            self.scales = torch.ones((cfg.n_layers, 2, num_pages, hkv, cfg.page_size), dtype=torch.float32,
                                     device=device)
        self.k_static, self.v_static = (k_static or 1.0, v_static or 1.0) if fmt == "fp8-static" else (0.0, 0.0)
        if static_scales is None and fmt == "fp8-static" and cfg.kv_static_scales:
            static_scales = [tuple(x) for x in cfg.kv_static_scales]     # the binding a converted checkpoint carries
        if static_scales is not None:
            if fmt != "fp8-static" or len(static_scales) != cfg.n_layers or any(k <= 0 or v <= 0 for k, v in static_scales):
                raise ValueError("static_scales needs the fp8-static format and one positive (k, v) pair per layer")
        per_layer = static_scales or [(self.k_static, self.v_static)] * cfg.n_layers
        self._layers = [
            KVLayer(self.values[l, 0], self.values[l, 1],
                    None if self.scales is None else self.scales[l, 0],
                    None if self.scales is None else self.scales[l, 1],
                    self.fp8, cfg.page_size, float(per_layer[l][0]), float(per_layer[l][1]), self.nvfp4)
            for l in range(cfg.n_layers)
        ]

    def layer(self, i: int) -> KVLayer:
        return self._layers[i]

    def bytes_per_token(self) -> int:
        s = self.spec
        b = 2 * s.n_layers * s.kv_heads * self.values.shape[-1] * self.values.element_size()
        if self.scales is not None:
            b += 2 * s.n_layers * s.kv_heads * 4
        return b

    def copy_page(self, src: int, dst: int) -> None:
        """Device copy of one page across all layers (fork tail / copy-on-write)."""
        self.values[:, :, dst].copy_(self.values[:, :, src])
        if self.scales is not None:
            self.scales[:, :, dst].copy_(self.scales[:, :, src])

    def fork(self, seq: int, prefix_len: int) -> int:
        child, (src, dst) = self.pool.fork(seq, prefix_len)
        if src >= 0:
            self.copy_page(src, dst)
        return child

    def ensure_private_tail(self, seq: int) -> None:
        pair = self.pool.make_tail_private(seq)
        if pair is not None:
            self.copy_page(*pair)

    def export_pages(self, seq: int) -> dict:
        """Raw page contents of one sequence (native encoding), for checkpoints."""
        pages = torch.tensor(self.pool.pages(seq), dtype=torch.long, device=self.device)
        out = {"values": self.values[:, :, pages].cpu(), "length": self.pool.length(seq)}
        if self.scales is not None:
            out["scales"] = self.scales[:, :, pages].cpu()
        return out

    def export_token_major(self, seqs: list, max_tokens: int) -> torch.Tensor:
        """Value planes of ``seqs`` in the reference's dense token-major order
        ``[layers, 2 (K, V), batch, blocks, block_size, kv_heads, head_dim]`` (docs/architecture/kv-memory.md of the
        reference; offsets as in its layout oracle tests/reference/oracles.py:209-239), blocks = ceil(max_tokens /
        page).  The resident pages are head-major (one head's 16 tokens contiguous); this is the interchange view for
        tools that expect the reference's order.  Tokens beyond a sequence's length read as zero."""
        page = self.pool.page_size
        blocks = (max_tokens + page - 1) // page
        L, two, _, hkv, _, hd = self.values.shape
        out = torch.zeros((L, two, len(seqs), blocks, page, hkv, hd), dtype=self.values.dtype, device=self.values.device)
        for bi, seq in enumerate(seqs):
            pages = self.pool.pages(seq)[:blocks]
            if pages:
                idx = torch.tensor(pages, dtype=torch.long, device=self.device)
                # [L, 2, n, hkv, page, hd] -> [L, 2, n, page, hkv, hd]
                out[:, :, bi, :len(pages)] = self.values[:, :, idx].permute(0, 1, 2, 4, 3, 5)
        return out

    def import_pages(self, image: dict) -> int:
        seq = self.pool.new_seq()
        n = int(image["length"])
        try:
            self.pool.reserve(seq, n)
        except Exception:
            self.pool.free_seq(seq)
            raise
        pages = torch.tensor(self.pool.pages(seq), dtype=torch.long, device=self.device)
        self.values[:, :, pages] = image["values"].to(self.device)
        if self.scales is not None:
            self.scales[:, :, pages] = image["scales"].to(self.device)
        self.pool.commit(seq, n)
        return seq

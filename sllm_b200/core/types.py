"""Scalar storage types, quantisation encodings and non-owning tensor views.

`DType` is the physical scalar; `Encoding` says how logical values map to stored scalars (unquantised, FP8 with
separately resident scales at tensor / outer-row / K-block granularity, NVFP4 and MXFP4 packed nibbles with block
scales, each in a weight-only W4A16 and a W4A4 form so that one is never selected for the other).  `TensorView`
describes a strided region of a buffer; launch wrappers use it to reject outputs that alias an input they may not alias.

Reference: crates/sllm-core/src/dtype.rs:6-130 (DType, Encoding, Fp8ScaleGranularity), tensor.rs:7-170 (TensorView).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Optional


class TensorError(ValueError):
    pass


class DType(enum.Enum):
    BF16 = ("bf16", 2, True)
    F16 = ("f16", 2, True)
    F32 = ("f32", 4, True)
    F8E4M3FN = ("f8e4m3fn", 1, True)
    F8E4M3FNUZ = ("f8e4m3fnuz", 1, True)
    F8E5M2 = ("f8e5m2", 1, True)
    F8E5M2FNUZ = ("f8e5m2fnuz", 1, True)
    I32 = ("i32", 4, False)
    I64 = ("i64", 8, False)
    I8 = ("i8", 1, False)
    U8 = ("u8", 1, False)

    def __str__(self) -> str:
        return self.value[0]

    @property
    def size_bytes(self) -> int:
        return self.value[1]

    @property
    def is_float(self) -> bool:
        return self.value[2]

    @staticmethod
    def parse(name: str) -> "DType":
        for d in DType:
            if d.value[0] == name:
                return d
        raise TensorError(f"unknown dtype {name!r}")

    @staticmethod
    def of_torch(dt) -> "DType":
        import torch
        table = {torch.bfloat16: DType.BF16, torch.float16: DType.F16, torch.float32: DType.F32, torch.int32: DType.I32,
                 torch.int64: DType.I64, torch.int8: DType.I8, torch.uint8: DType.U8}
        if hasattr(torch, "float8_e4m3fn"):
            table[torch.float8_e4m3fn] = DType.F8E4M3FN
            table[torch.float8_e5m2] = DType.F8E5M2
        if dt not in table:
            raise TensorError(f"torch dtype {dt} has no storage type here")
        return table[dt]


class Fp8ScaleGranularity(enum.Enum):
    TENSOR = "tensor"                 # one scale for the whole tensor (static KV scales)
    OUTER_DIMENSION = "outer"         # one scale per row of a row-major matrix (channel scales; per-token activations)
    K_BLOCK = "kblock"                # one scale per consecutive K block in every row (block 128: the resident form)


class EncodingKind(enum.Enum):
    UNQUANTIZED = "unquantized"
    FP8_SCALED = "fp8-scaled"
    NVFP4 = "nvfp4"                   # weight-only (W4A16): E2M1 nibbles, E4M3 scale per 16, FP32 tensor scale
    NVFP4_W4A4 = "nvfp4-w4a4"
    MXFP4 = "mxfp4"                   # weight-only (W4A16): E2M1 nibbles, E8M0 scale per 32
    MXFP4_W4A4 = "mxfp4-w4a4"


@dataclass(frozen=True)
class Encoding:
    kind: EncodingKind
    block_size: int = 0
    scale_dtype: Optional[DType] = None
    granularity: Optional[Fp8ScaleGranularity] = None

    @staticmethod
    def unquantized() -> "Encoding":
        return Encoding(EncodingKind.UNQUANTIZED)

    @staticmethod
    def fp8(granularity: Fp8ScaleGranularity, block_size: int = 0, scale_dtype: DType = DType.F32) -> "Encoding":
        return Encoding(EncodingKind.FP8_SCALED, block_size, scale_dtype, granularity)

    @staticmethod
    def nvfp4(w4a4: bool = False) -> "Encoding":
        return Encoding(EncodingKind.NVFP4_W4A4 if w4a4 else EncodingKind.NVFP4, 16, DType.F8E4M3FN)

    @staticmethod
    def mxfp4(w4a4: bool = False) -> "Encoding":
        return Encoding(EncodingKind.MXFP4_W4A4 if w4a4 else EncodingKind.MXFP4, 32, DType.U8)

    @staticmethod
    def of_weight_format(name: str) -> "Encoding":
        """The resident encoding of a model's `weight_format`."""
        if name in ("fp32", "bf16", "fp16"):
            return Encoding.unquantized()
        if name == "fp8":
            return Encoding.fp8(Fp8ScaleGranularity.K_BLOCK, 128)
        if name == "nvfp4":
            return Encoding.nvfp4()
        if name == "mxfp4":
            return Encoding.mxfp4()
        raise TensorError(f"unknown weight format {name!r}")

    @staticmethod
    def of_kv_format(name: str) -> "Encoding":
        if name in ("fp32", "bf16", "fp16"):
            return Encoding.unquantized()
        if name == "fp8":
            return Encoding.fp8(Fp8ScaleGranularity.OUTER_DIMENSION)      # one scale per (token, head) row
        if name == "fp8-static":
            return Encoding.fp8(Fp8ScaleGranularity.TENSOR)
        if name == "nvfp4":
            return Encoding(EncodingKind.NVFP4, 16, DType.F8E4M3FN)
        raise TensorError(f"unknown KV format {name!r}")

    def validate(self, dtype: DType) -> None:
        k = self.kind
        if k is EncodingKind.UNQUANTIZED:
            if self.block_size or self.scale_dtype or self.granularity:
                raise TensorError("an unquantised encoding carries no block or scale description")
            return
        if k is EncodingKind.FP8_SCALED:
            if dtype not in (DType.F8E4M3FN, DType.F8E4M3FNUZ, DType.F8E5M2, DType.F8E5M2FNUZ, DType.U8):
                raise TensorError(f"FP8 values are stored as one byte, not {dtype}")
            if self.granularity is None or self.scale_dtype not in (DType.F32, DType.BF16):
                raise TensorError("FP8 needs a scale granularity and F32 or BF16 scales")
            if (self.granularity is Fp8ScaleGranularity.K_BLOCK) != (self.block_size > 0):
                raise TensorError("a block size goes with the K-block granularity and with nothing else")
            return
        if dtype is not DType.U8:
            raise TensorError("packed four-bit values are stored as bytes")
        want = (16, DType.F8E4M3FN) if k in (EncodingKind.NVFP4, EncodingKind.NVFP4_W4A4) else (32, DType.U8)
        if (self.block_size, self.scale_dtype) != want:
            raise TensorError(f"{k.value}: block {want[0]} with {want[1]} scales")

    def offset_alignment(self, dtype: DType) -> int:
        return dtype.size_bytes if self.kind is EncodingKind.UNQUANTIZED else 16

    def payload_bytes(self, dtype: DType, elements: int) -> int:
        """Bytes of the value payload of `elements` logical values (scales live elsewhere)."""
        if self.kind in (EncodingKind.UNQUANTIZED, EncodingKind.FP8_SCALED):
            return elements * dtype.size_bytes
        return (elements + 1) // 2


@dataclass(frozen=True)
class TensorView:
    """Strided region of a buffer: strides in logical elements, offset in bytes from the buffer's base."""
    dtype: DType
    shape: tuple
    strides: tuple
    byte_offset: int = 0
    encoding: Encoding = Encoding(EncodingKind.UNQUANTIZED)
    base: int = 0                    # address of the backing buffer (0 for a descriptor without storage)

    def __post_init__(self):
        if len(self.shape) != len(self.strides):
            raise TensorError(f"rank mismatch: shape {len(self.shape)}, strides {len(self.strides)}")
        if any(int(s) < 0 for s in self.shape) or any(int(s) < 0 for s in self.strides):
            raise TensorError("negative extent or stride")
        self.encoding.validate(self.dtype)
        if self.byte_offset % self.encoding.offset_alignment(self.dtype):
            raise TensorError(f"offset {self.byte_offset} is not aligned to {self.encoding.offset_alignment(self.dtype)}")
        if self.encoding.kind not in (EncodingKind.UNQUANTIZED, EncodingKind.FP8_SCALED) and not self.is_contiguous:
            raise TensorError("packed encodings need a contiguous view")
        if self.span_bytes > (1 << 62):
            raise TensorError("shape overflow")

    @staticmethod
    def contiguous(dtype: DType, shape, encoding: Optional[Encoding] = None, base: int = 0) -> "TensorView":
        strides, run = [], 1
        for s in reversed(tuple(shape)):
            strides.append(run)
            run *= int(s)
        return TensorView(dtype, tuple(int(s) for s in shape), tuple(reversed(strides)), 0,
                          encoding or Encoding.unquantized(), base)

    @property
    def element_count(self) -> int:
        n = 1
        for s in self.shape:
            n *= int(s)
        return n

    @property
    def is_contiguous(self) -> bool:
        run = 1
        for s, st in zip(reversed(self.shape), reversed(self.strides)):
            if s != 1 and st != run:
                return False
            run *= int(s)
        return True

    @property
    def span_bytes(self) -> int:
        """Bytes from the first to one past the last addressed value."""
        if self.element_count == 0:
            return 0
        last = sum((int(s) - 1) * int(st) for s, st in zip(self.shape, self.strides))
        return self.encoding.payload_bytes(self.dtype, last + 1)

    @property
    def begin(self) -> int:
        return self.base + self.byte_offset

    @property
    def end(self) -> int:
        return self.begin + self.span_bytes

    def overlaps(self, other: "TensorView") -> bool:
        """True when the two views address at least one common byte of storage (both must carry a base address)."""
        if not self.base or not other.base or self.span_bytes == 0 or other.span_bytes == 0:
            return False
        return self.begin < other.end and other.begin < self.end

    def same_region(self, other: "TensorView") -> bool:
        return self.begin == other.begin and self.shape == other.shape and self.strides == other.strides and \
            self.dtype == other.dtype


def view_of(t, encoding: Optional[Encoding] = None) -> TensorView:
    """The view of a torch tensor's storage."""
    return TensorView(DType.of_torch(t.dtype), tuple(t.shape), tuple(t.stride()), 0, encoding or Encoding.unquantized(),
                      t.data_ptr())


def _byte_span(t) -> tuple:
    """[begin, end) of the bytes a torch tensor addresses (no object construction: this runs on every GEMM launch)."""
    n = t.numel()
    if n == 0:
        return 0, 0
    b = t.data_ptr()
    if t.is_contiguous():
        return b, b + n * t.element_size()
    last = 0
    for s_, st in zip(t.shape, t.stride()):
        last += (s_ - 1) * st
    return b, b + (last + 1) * t.element_size()


def reject_aliasing(out, inputs: dict, may_equal: tuple = ()) -> None:
    """Raises TensorError when `out` overlaps one of `inputs` (name -> tensor or None).  Inputs named in `may_equal`
    may BE the output (the same region: an in-place residual), but may not overlap it partially."""
    ob, oe = _byte_span(out)
    for name, t in inputs.items():
        if t is None:
            continue
        ib, ie = _byte_span(t)
        if ib >= oe or ob >= ie or ib == ie or ob == oe:
            continue
        if name in may_equal and ib == ob and t.shape == out.shape and t.stride() == out.stride() and t.dtype == out.dtype:
            continue
        raise TensorError(f"the output overlaps input {name!r} (bytes [{ib:#x}, {ie:#x}) vs [{ob:#x}, {oe:#x}))")

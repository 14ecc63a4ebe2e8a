"""Core contracts: storage types and encodings, tensor views (strides, spans, overlap), alias rejection at the GEMM entry
points, the backend registry and its fake."""
import pytest
import torch

from sllm_b200 import core as C
from sllm_b200.core.types import reject_aliasing


def test_dtype_and_encoding_rules():
    assert C.DType.parse("f8e4m3fn").size_bytes == 1 and C.DType.BF16.is_float and not C.DType.I32.is_float
    assert str(C.DType.F8E4M3FNUZ) == "f8e4m3fnuz"
    with pytest.raises(C.TensorError):
        C.DType.parse("f7")
    e = C.Encoding.of_weight_format("fp8")
    assert e.granularity is C.Fp8ScaleGranularity.K_BLOCK and e.block_size == 128
    assert C.Encoding.of_kv_format("fp8-static").granularity is C.Fp8ScaleGranularity.TENSOR
    assert C.Encoding.of_kv_format("fp8").granularity is C.Fp8ScaleGranularity.OUTER_DIMENSION
    assert C.Encoding.nvfp4().kind is not C.Encoding.nvfp4(w4a4=True).kind        # W4A16 is never taken for W4A4
    assert C.Encoding.mxfp4().block_size == 32 and C.Encoding.nvfp4().scale_dtype is C.DType.F8E4M3FN
    C.Encoding.of_weight_format("nvfp4").validate(C.DType.U8)
    for enc, dt in ((C.Encoding.nvfp4(), C.DType.BF16), (C.Encoding.fp8(C.Fp8ScaleGranularity.K_BLOCK, 0), C.DType.U8),
                    (C.Encoding.fp8(C.Fp8ScaleGranularity.TENSOR, 128), C.DType.U8),
                    (C.Encoding.fp8(C.Fp8ScaleGranularity.TENSOR), C.DType.F32),
                    (C.Encoding(C.EncodingKind.NVFP4, 32, C.DType.U8), C.DType.U8)):
        with pytest.raises(C.TensorError):
            enc.validate(dt)
    assert C.Encoding.nvfp4().payload_bytes(C.DType.U8, 33) == 17


def test_tensor_views_and_overlap():
    v = C.TensorView.contiguous(C.DType.BF16, (4, 8), base=0x1000)
    assert v.strides == (8, 1) and v.is_contiguous and v.span_bytes == 64 and v.element_count == 32
    row = C.TensorView(C.DType.BF16, (4, 4), (8, 1), 8, base=0x1000)           # the right half of every row
    assert not row.is_contiguous and row.span_bytes == (3 * 8 + 3 + 1) * 2 and row.overlaps(v)
    far = C.TensorView.contiguous(C.DType.BF16, (4, 8), base=0x1000 + 64)
    assert not far.overlaps(v) and not v.overlaps(far)
    with pytest.raises(C.TensorError):
        C.TensorView(C.DType.BF16, (4, 8), (8,))
    with pytest.raises(C.TensorError):
        C.TensorView(C.DType.F32, (4,), (1,), 2)                                    # misaligned offset
    with pytest.raises(C.TensorError):
        C.TensorView(C.DType.U8, (4, 8), (16, 1), 0, C.Encoding.nvfp4())          # packed views are contiguous
    t = torch.zeros(6, 10)
    a, b = t[:4], t[2:]
    assert C.view_of(a).overlaps(C.view_of(b)) and not C.view_of(t[:2]).overlaps(C.view_of(t[4:]))
    reject_aliasing(t[:2], {"x": t[4:], "residual": t[:2]}, may_equal=("residual",))
    with pytest.raises(C.TensorError):
        reject_aliasing(a, {"x": b})
    with pytest.raises(C.TensorError):
        reject_aliasing(a, {"residual": b}, may_equal=("residual",))               # partial overlap is never allowed


def test_backend_registry_and_fake():
    assert set(C.BACKENDS) == {"fake", "cuda-sm100a"}
    with pytest.raises(C.BackendError):
        C.create_backend("rocm")
    fake = C.create_backend("fake")
    caps = fake.capabilities()
    assert caps.metadata_only and not caps.numerical_execution and caps.max_materialization_bytes == 1 << 30
    assert fake.supports("linear") is None and fake.supports("fft") is not None
    m = fake.materialize(C.TensorView.contiguous(C.DType.BF16, (8, 8)))
    assert m["metadata_only"] and m["byte_len"] == 128
    with pytest.raises(C.BackendError):
        fake.materialize(C.TensorView.contiguous(C.DType.F32, (1 << 20, 1 << 10)))
    with pytest.raises(C.BackendError):
        fake.execute("linear", x=C.TensorView.contiguous(C.DType.BF16, (2, 4)))
    with pytest.raises(C.BackendError):
        fake.execute("linear", x=C.TensorView.contiguous(C.DType.BF16, (0, 4)))
    assert [e[0] for e in fake.log] == ["materialize", "execute"]
    cuda = C.create_backend("cuda-sm100a")
    if not torch.cuda.is_available():
        assert cuda.available() is not None and not cuda.capabilities().numerical_execution
        assert cuda.supports("linear") is not None
        with pytest.raises(C.BackendError):
            cuda.execute("rmsnorm", x=torch.zeros(2, 8), weight=torch.ones(8), eps=1e-5)     # unavailable: never computes
    assert "nvfp4" in cuda.capabilities().kv_formats and "peer-memory" in cuda.capabilities().collective_backends


@pytest.mark.gpu
def test_gemm_entry_points_reject_aliased_outputs():
    from sllm_b200 import ops
    x = torch.randn(32, 256, device="cuda").bfloat16()
    w = torch.randn(256, 256, device="cuda").bfloat16()
    with pytest.raises(C.TensorError):
        ops.gemm_raw(w, x, x[:, :256], transpose_out=True, bn=32, splits=1, stages=4)      # output = the activation operand
    y = torch.empty(32, 256, device="cuda", dtype=torch.bfloat16)
    ops.gemm_raw(w, x, y, residual=y, transpose_out=True, bn=32, splits=1, stages=4)       # in-place residual is allowed
    assert ops.device_status(torch.device("cuda")) == 0

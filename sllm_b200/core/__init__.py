"""Core contracts: scalar / encoding types, non-owning tensor views with overlap checks, and the backend registry."""
from .types import DType, Encoding, EncodingKind, Fp8ScaleGranularity, TensorError, TensorView, view_of  # noqa: F401
from .backends import BACKENDS, Backend, BackendCapabilities, BackendError, CudaBackend, FakeBackend, create_backend  # noqa: F401

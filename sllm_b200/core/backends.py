"""Backend contract and the static registry.

A backend says what it can do (`capabilities`), whether it supports a semantic op, and either computes or refuses.
Two are registered: `cuda-sm100a` (the kernel library: numerical execution on a B200; unavailable - never computing -
where no such GPU or no built library exists) and `fake` (metadata only: validates views and ops, records what it was
asked, executes nothing; the double the contract tests run against).

Reference: crates/sllm-core/src/backend.rs:9-100 (Backend, BackendCapabilities, BackendSupport, ExecutionReceipt,
BackendError), registry.rs (static registry, no dynamic loading), fake.rs.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

from .types import TensorError, TensorView

# semantic ops of the graph builders (reference: crates/sllm-core/src/op.rs SemanticOpKind)
SEMANTIC_OPS = ("embedding", "rmsnorm", "linear", "rotary", "kv_append", "attention", "gated_activation", "elementwise_add",
                "scalar_mul", "softcap", "moe_route", "moe_experts", "moe_combine", "gated_delta_net", "causal_conv",
                "token_select", "final_output")


class BackendError(RuntimeError):
    pass


@dataclass(frozen=True)
class BackendCapabilities:
    metadata_only: bool
    numerical_execution: bool
    max_materialization_bytes: Optional[int]
    weight_formats: tuple = ()
    kv_formats: tuple = ()
    collective_backends: tuple = ()


class Backend:
    name = "abstract"

    def capabilities(self) -> BackendCapabilities:
        raise NotImplementedError

    def supports(self, op: str) -> Optional[str]:
        """None when the op is supported, else the reason it is not."""
        raise NotImplementedError

    def materialize(self, view: TensorView) -> dict:
        raise NotImplementedError

    def execute(self, op: str, **operands) -> dict:
        raise NotImplementedError


@dataclass
class FakeBackend(Backend):
    """Validates and records; computes nothing."""
    name: str = "fake"
    max_bytes: int = 1 << 30
    log: list = field(default_factory=list)

    def capabilities(self) -> BackendCapabilities:
        return BackendCapabilities(True, False, self.max_bytes)

    def supports(self, op: str) -> Optional[str]:
        return None if op in SEMANTIC_OPS else "unknown semantic op"

    def materialize(self, view: TensorView) -> dict:
        if view.span_bytes > self.max_bytes:
            raise BackendError(f"metadata materialization requested {view.span_bytes} bytes, limit is {self.max_bytes}")
        self.log.append(("materialize", view.shape, str(view.dtype)))
        return {"metadata_only": True, "byte_len": view.span_bytes, "view": view}

    def execute(self, op: str, **operands) -> dict:
        why = self.supports(op)
        if why:
            raise BackendError(f"operation {op} is unsupported: {why}")
        for name, v in operands.items():
            if isinstance(v, TensorView) and v.element_count == 0:
                raise BackendError(f"invalid tensor: operand {name} is empty")
        self.log.append(("execute", op, tuple(sorted(operands))))
        raise BackendError("numerical execution is unavailable on the fake backend")


class CudaBackend(Backend):
    """The sm_100a kernel library.  `available()` is false (and nothing computes) without a GPU or a built library."""
    name = "cuda-sm100a"

    def available(self) -> Optional[str]:
        from ..ops import _lib
        try:
            import torch
        except ImportError:
            return "torch is not importable"
        if not _lib.kernels_available():
            return "the kernel library has not been built"
        if not torch.cuda.is_available():
            return "no CUDA device"
        if torch.cuda.get_device_capability(0)[0] != 10:
            return "the kernels are built for sm_100a only"
        return None

    def capabilities(self) -> BackendCapabilities:
        ok = self.available() is None
        return BackendCapabilities(False, ok, None, ("bf16", "fp8", "nvfp4", "mxfp4"),
                                   ("bf16", "fp8", "fp8-static", "nvfp4"), ("peer-memory", "nccl"))

    def supports(self, op: str) -> Optional[str]:
        if op not in SEMANTIC_OPS:
            return "unknown semantic op"
        return self.available()

    def materialize(self, view: TensorView) -> dict:
        why = self.available()
        if why:
            raise BackendError(f"backend {self.name} is unavailable: {why}")
        import torch
        n = view.span_bytes
        buf = torch.empty(n, dtype=torch.uint8, device="cuda")
        return {"metadata_only": False, "byte_len": n, "buffer": buf, "view": view}

    def execute(self, op: str, **operands) -> dict:
        why = self.supports(op)
        if why:
            raise BackendError(f"backend {self.name} is unavailable: {why}")
        from .. import ops
        table = {"rmsnorm": ops.rmsnorm, "linear": ops.linear, "gated_activation": ops.gated_act, "embedding": ops.embedding,
                 "token_select": ops.argmax}
        if op not in table:
            raise BackendError(f"operation {op} runs through the model graph, not through single-op execution")
        return {"operation": op, "result": table[op](**operands)}


BACKENDS: dict = {"fake": FakeBackend, "cuda-sm100a": CudaBackend}      # static: no dynamic plug-in loading


def create_backend(name: str) -> Backend:
    if name not in BACKENDS:
        raise BackendError(f"backend {name} is unavailable")
    return BACKENDS[name]()

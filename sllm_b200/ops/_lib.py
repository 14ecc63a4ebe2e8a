"""ctypes bindings for the two native libraries.

``kernels()`` loads ``libsllm_b200_kernels.so`` (CUDA, sm_100a) and raises if it is missing: there is
no silent fallback to PyTorch on a GPU.  ``host()`` loads ``libsllm_b200_host.so`` (pure C++).
Signatures are declared once here from ``csrc/api.h`` / ``csrc/host/host_api.h``.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Optional
from pathlib import Path

_PKG = Path(__file__).resolve().parent.parent
_KERNEL_PATH = _PKG / "libsllm_b200_kernels.so"
_HOST_PATH = _PKG / "libsllm_b200_host.so"
_lock = threading.Lock()
_kernels = None
_host = None

P = C.c_void_p
I = C.c_int
L = C.c_longlong
F = C.c_float

STATUS_NAMES = {
    0: "ok", 1: "invalid argument", 2: "unsupported shape", 3: "alignment", 4: "workspace too small",
    5: "cuda error", 6: "driver entry point unavailable", 7: "limit exceeded",
}
DEVICE_STATUS_NAMES = {
    0: "ok", 101: "timeout waiting for TMA data", 102: "timeout waiting for a free smem stage",
    103: "timeout waiting for the accumulator", 104: "timeout waiting for a free accumulator",
    105: "timeout waiting for a peer flag", 106: "timeout draining copies",
    107: "timeout waiting at a grid barrier",
}


class KernelError(RuntimeError):
    pass


LAUNCH_COUNT = [0]  # kernels launched through this library (graph capture counts once per capture)

# Work that left its intended fast path, by reason (reported by /props and the benchmark line; the reference's
# dispatch records carry the same information as `fallback_used`, include/sllm/hip.h:651-671).
FALLBACKS: dict = {}


def note_fallback(reason: str) -> None:
    FALLBACKS[reason] = FALLBACKS.get(reason, 0) + 1


def fallbacks() -> dict:
    return dict(FALLBACKS)


# Fail-closed mode: with it on, an op that is handed a CPU tensor raises instead of computing the PyTorch oracle of
# the op (the reference's host build of its native layer reports "unavailable" and never computes:
# native/hip/src/host_stub.cpp).  On by SLLM_FAIL_CLOSED=1 or set_fail_closed(True); the server switches it on when it
# serves from a GPU, so a tensor that strays to the CPU is an error there and not a silent slow path.
_fail_closed = [None]


def set_fail_closed(on: bool) -> None:
    _fail_closed[0] = bool(on)


def fail_closed() -> bool:
    if _fail_closed[0] is None:
        import os
        _fail_closed[0] = os.environ.get("SLLM_FAIL_CLOSED", "0") == "1"
    return _fail_closed[0]


_cuda_present = [None]


def on_cpu(t) -> bool:
    """True when the op should take its CPU oracle branch for tensor ``t``.  Raises in fail-closed mode; on a machine
    that has a GPU the detour is recorded as a fallback."""
    if t.is_cuda or _fake[0] is not None:
        return False
    if fail_closed():
        raise KernelError("CUDA kernels are required (fail-closed mode): the op was handed a CPU tensor")
    if _cuda_present[0] is None:
        import torch
        _cuda_present[0] = torch.cuda.is_available()
    if _cuda_present[0]:
        note_fallback("cpu_oracle_on_gpu_host")
    return True


# Dispatch audit: when switched on, every planned launch of the main ops leaves a record (op, kernel path, shape,
# tile / split plan, whether the fast path was left) in a bounded ring that /props, the evidence runners and tests
# read (reference: the dispatch-info records of include/sllm/hip.h:651-671 - kernel id, grid, fallback_used).
_AUDIT_CAP = 256
_audit_on = [None]
_audit_ring: list = []
_audit_total = [0]


def audit(on: bool) -> None:
    _audit_on[0] = bool(on)


def audit_enabled() -> bool:
    if _audit_on[0] is None:
        import os
        _audit_on[0] = os.environ.get("SLLM_DISPATCH_AUDIT", "0") == "1"
    return _audit_on[0]


def record_dispatch(op: str, kernel: str, fallback_used: bool = False, **info) -> None:
    if not audit_enabled():
        return
    _audit_total[0] += 1
    _audit_ring.append({"seq": _audit_total[0], "op": op, "kernel": kernel, "fallback_used": bool(fallback_used), **info})
    if len(_audit_ring) > _AUDIT_CAP:
        del _audit_ring[:len(_audit_ring) - _AUDIT_CAP]


def dispatch_records(clear: bool = False) -> list:
    out = list(_audit_ring)
    if clear:
        _audit_ring.clear()
    return out


# Per-launch device timing (eager launches only): with timing on, every successful launch is followed by a CUDA event
# on the current stream; the report gives, per launch, the device time since the previous event.
_timing: list = []
_timing_on = [False]


def timing(on: bool) -> None:
    """Starts (records the base event) or stops per-launch timing.  Not usable during stream capture."""
    import torch
    _timing_on[0] = bool(on) and torch.cuda.is_available() and not fake_active()
    _timing.clear()
    if _timing_on[0]:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        _timing.append(("<start>", ev))


def timing_report() -> list:
    """[(launch name, microseconds since the previous launch finished)] since `timing(True)`; synchronises."""
    import torch
    if len(_timing) < 2:
        return []
    torch.cuda.synchronize()
    return [(name, _timing[i - 1][1].elapsed_time(ev) * 1e3) for i, (name, ev) in enumerate(_timing) if i > 0]


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what}: launch rejected ({STATUS_NAMES.get(rc, rc)})")
    LAUNCH_COUNT[0] += 1
    if _timing_on[0]:
        import torch
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        _timing.append((what, ev))


_KERNEL_SIGNATURES = {
    "sllm_gemm_workspace_floats": (L, [I, I, I, I]),
    "sllm_gemm": (I, [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, L, P, I, P, P]),
    "sllm_embedding": (I, [P, P, P, I, I, I, F, P]),
    "sllm_rmsnorm": (I, [P, P, P, P, P, I, I, I, F, I, P]),
    "sllm_gated_act": (I, [P, P, P, P, I, I, I, I, P]),
    "sllm_quant_fp8_1x128": (I, [P, P, P, I, I, I, P]),
    "sllm_rope_kv_append": (I, [P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, F, F, F, P, P]),
    "sllm_rope_kv_append_paired": (I, [P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, F, F, F, P, I, P]),
    "sllm_rope_kv_append_mrope": (I, [P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, F, F, F, P, P, I, I, P]),
    "sllm_elementwise": (I, [P, P, P, L, I, I, F, P]),
    "sllm_argmax": (I, [P, P, P, I, I, I, I, P, L, P, I, P]),
    "sllm_gemm_set_cluster_split": (None, [I]),
    "sllm_decode_attention_tc": (I, [P, I, P, P, P, P, F, F, P, I, P, P, I, I, I, I, I, I, F, P, P, P, I, P, I, P, L,
                                      P, I, P, P]),
    "sllm_prefill_attention": (I, [P, I, I, P, I, I, I, I, F, P, P, P, I, P, P]),
    "sllm_paged_attention_workspace_floats": (L, [I, I, I, I, I]),
    "sllm_paged_attention": (I, [P, I, P, P, P, P, F, F, P, I, P, P, I, I, I, I, I, I, F, I, P, P, P, I, P, I, P, L,
                                  P, I, P]),
}

# Entry points added by later translation units register themselves here (name -> (restype, argtypes)).
EXTRA_KERNEL_SIGNATURES: dict = {}


def kernels_available() -> bool:
    return _KERNEL_PATH.exists()


# ---------------------------------------------------------------------------------------------- fake device layer
class FakeKernelLibrary:
    """Programmable stand-in for the kernel library (reference: native/hip/tests/fake_hip/fake_hip_runtime.cpp).

    Every entry point of the signature tables exists; a call is recorded as (name, args) and returns the next status
    scripted for that name (`script = {"sllm_gemm": [0, 0, 9]}`: the third GEMM launch is rejected with status 9;
    an exhausted or missing script means 0).  Nothing is computed and no pointer is dereferenced, so it runs on a
    machine without a GPU: while a fake is installed the ops take their device branch for CPU tensors too (outputs are
    allocated but not written).  Used to test what the layers above do with launch failures."""

    def __init__(self, script: Optional[dict] = None):
        self.script = {k: list(v) for k, v in (script or {}).items()}
        self.calls: list = []

    def __getattr__(self, name: str):
        if name.startswith("__") or (name not in _KERNEL_SIGNATURES and name not in EXTRA_KERNEL_SIGNATURES):
            raise AttributeError(name)
        restype = (_KERNEL_SIGNATURES.get(name) or EXTRA_KERNEL_SIGNATURES.get(name))[0]

        def call(*args):
            self.calls.append((name, args))
            if restype is None:
                return None
            pending = self.script.get(name)
            return pending.pop(0) if pending else 0
        return call

    def count(self, name: str) -> int:
        return sum(1 for n, _ in self.calls if n == name)


_fake = [None]


def install_fake(fake: Optional[FakeKernelLibrary]) -> None:
    """Routes every kernel call to `fake` (None restores the real library)."""
    _fake[0] = fake


def fake_active() -> bool:
    return _fake[0] is not None


def kernels():
    """The CUDA kernel library.  Raises when it has not been built."""
    global _kernels
    if _fake[0] is not None:
        return _fake[0]
    if _kernels is None:
        with _lock:
            if _kernels is None:
                if not _KERNEL_PATH.exists():
                    raise KernelError(
                        f"{_KERNEL_PATH.name} is missing: run `python -m sllm_b200.build` (nvcc, sm_100a); "
                        "CUDA tensors are never routed to a PyTorch fallback")
                lib = C.CDLL(str(_KERNEL_PATH))
                _apply(lib, _KERNEL_SIGNATURES)
                _kernels = lib
    if len(_applied) < len(_KERNEL_SIGNATURES) + len(EXTRA_KERNEL_SIGNATURES):
        _apply(_kernels, EXTRA_KERNEL_SIGNATURES)
    return _kernels


_applied: set = set()


def _apply(lib, table: dict) -> None:
    for name, (res, args) in table.items():
        if name not in _applied and hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _applied.add(name)


def host():
    """The host runtime library (page pool, grammar, sampler chain, batch planner)."""
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                if not _HOST_PATH.exists():
                    from .. import build
                    build.build_host()
                _host = C.CDLL(str(_HOST_PATH))
    return _host

"""Descriptor structs mirrored by hand in ctypes agree with the layout the native library was compiled with."""
import pytest

from sllm_b200.ops import _lib

pytestmark = pytest.mark.skipif(not _lib.kernels_available(), reason="kernel library not built")


def test_communicator_and_fused_decode_descriptor_layouts():
    from sllm_b200.ops import fused_decode as fd
    from sllm_b200.parallel import tp
    tp._abi_ok = False
    fd._abi_checked = False
    tp.check_comm_abi()
    fd.check_abi()
    assert tp._abi_ok and fd._abi_checked


def test_a_drifted_mirror_is_refused(monkeypatch):
    import ctypes as C
    from sllm_b200.parallel import tp

    class Drifted(C.Structure):       # two fields swapped
        _fields_ = [("rank", C.c_int), ("world", C.c_int), ("cap_elems", C.c_longlong), ("max_tiles", C.c_int),
                    ("reserved", C.c_int), ("flags", C.c_void_p * 8), ("recv", C.c_void_p * 8), ("epoch", C.c_void_p)]

    monkeypatch.setattr(tp, "CommDesc", Drifted)
    tp._abi_ok = False
    with pytest.raises(_lib.KernelError):
        tp.check_comm_abi()
    tp._abi_ok = False


def test_host_sampler_struct_layouts(monkeypatch):
    """The sampler configuration / state mirrors are checked against the host library when it is first bound; a mirror
    with two fields swapped is refused."""
    import ctypes as C
    from sllm_b200.engine import sampling as S
    S._native["lib"] = None
    assert S._native_lib() is not None

    class Drifted(C.Structure):
        _fields_ = [("draws", C.c_longlong), ("rng_state", C.c_uint64), ("mu", C.c_double)]

    monkeypatch.setattr(S, "_NativeState", Drifted)
    S._native["lib"] = None
    with pytest.raises(S.SamplingError, match="layout mismatch"):
        S._native_lib()
    monkeypatch.undo()
    S._native["lib"] = None
    assert S._native_lib() is not None

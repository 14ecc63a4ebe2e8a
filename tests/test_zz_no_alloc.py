"""The allocation-free argmax entry point, called through its exported C symbol.

Some embedders may not allocate device memory at all (plug-ins under a foreign memory budget, components
whose allocations are frozen after start-up); for them the library keeps the scratch of this one
operation in a fixed device array.  The test checks that it returns exactly what the regular entry
point returns, twice in a row (the second call reuses the array the first one left behind), and that a
batch beyond the stated capacity is refused."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from sllm_b200.ops import _lib
    lib = _lib.kernels()
    lib.sllm_argmax_noalloc.restype = C.c_int
    lib.sllm_argmax_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.sllm_argmax_noalloc_max_rows.restype = C.c_int
    return lib


def test_noalloc_argmax_matches_regular_entry_point_twice():
    from sllm_b200 import ops
    lib = _lib()
    dev = torch.device("cuda")
    torch.manual_seed(123)
    for call, (rows, n) in enumerate([(32, 128256), (5, 4099)]):
        logits = torch.randn(rows, n, device=dev).bfloat16()
        logits[1, 17] = 60.0
        logits[1, n - 3] = 60.0          # tie -> lowest index
        if rows > 2:
            logits[2, 9] = float("nan")  # NaN row -> -1
        want_idx, want_val = ops.argmax(logits, index_offset=1000 * call, with_values=True)
        out_idx = torch.full((rows,), -7, dtype=torch.int32, device=dev)
        out_val = torch.zeros(rows, dtype=torch.float32, device=dev)
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.sllm_argmax_noalloc(logits.data_ptr(), out_idx.data_ptr(), out_val.data_ptr(), rows, n,
                                     logits.stride(0), 1000 * call, C.c_void_p(stream))
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(out_idx, want_idx)
        both = ~torch.isnan(want_val)
        assert torch.equal(out_val[both], want_val[both])
        assert out_idx[1].item() == 17 + 1000 * call
        # and, independently of this library's own kernel: rows without a tie or a NaN agree with torch.argmax
        plain = [r for r in range(rows) if r not in (1, 2)]
        assert torch.equal(out_idx[plain].long() - 1000 * call, logits[plain].float().argmax(dim=-1))
    too_many = lib.sllm_argmax_noalloc_max_rows() + 1
    big = torch.zeros(too_many, 16, device=dev, dtype=torch.bfloat16)
    out = torch.zeros(too_many, dtype=torch.int32, device=dev)
    rc = lib.sllm_argmax_noalloc(big.data_ptr(), out.data_ptr(), None, too_many, 16, 16, 0, None)
    assert rc == 7      # limit exceeded, nothing launched
    ok_rows = torch.zeros(4, 16, device=dev, dtype=torch.bfloat16)
    rc = lib.sllm_argmax_noalloc(ok_rows.data_ptr(), out.data_ptr(), None, 4, 16, 8, 0, None)
    assert rc == 1      # a row stride below the row length would make rows overlap

"""Failure paths made on the host (CPU) and bounded device waits that give up (GPU), without faulting anything."""
import ctypes as C

import pytest
import torch

from sllm_b200.cache.paged import OutOfPages
from sllm_b200.engine.engine import build_engine
from sllm_b200.models import config as MC


def test_injected_page_allocation_failure_fails_the_request_not_the_engine():
    """The page pool's fault hook makes one allocation fail: the step raises, the sequence's published state is
    untouched, and the same request succeeds afterwards with the result of an undisturbed engine."""
    cfg = MC.tiny_llama()
    prompt = list(range(3, 40))
    eng = build_engine(cfg, "cpu", seed=2, num_pages=64, max_batch=4, use_cuda_graphs=False)
    want = build_engine(cfg, "cpu", seed=2, num_pages=64, max_batch=4, use_cuda_graphs=False).generate([prompt], 5)[0]
    s = eng.new_sequence(prompt)
    free_before = eng.cache.pool.stats()["free"]
    eng.cache.pool.inject_alloc_failure(0)
    with pytest.raises(OutOfPages):
        eng.prefill([s])
    assert s.num_computed == 0 and eng.cache.pool.length(s.seq_id) == 0
    assert eng.cache.pool.stats()["free"] == free_before          # nothing leaked
    eng.cache.pool.inject_alloc_failure(-1)                       # the hook fails every allocation until it is cleared
    got = [eng.prefill([s])[0]]
    for _ in range(4):
        s.tokens.append(got[-1])
        got.append(eng.decode([s])[0])
    assert got == want
    # a failure in the middle of decoding: only that step fails
    s.tokens.append(got[-1])
    while eng.cache.pool.length(s.seq_id) % cfg.page_size != 0 or len(s.tokens) % cfg.page_size != 1:
        s.tokens.append(eng.decode([s])[0])                        # run up to a page boundary
    published = eng.cache.pool.length(s.seq_id)
    eng.cache.pool.inject_alloc_failure(0)
    with pytest.raises(OutOfPages):
        eng.decode([s])
    assert eng.cache.pool.length(s.seq_id) == published
    eng.cache.pool.inject_alloc_failure(-1)
    assert isinstance(eng.decode([s])[0], int)


@pytest.mark.gpu
def test_bounded_peer_wait_gives_up_and_the_context_survives():
    """A cross-rank sum whose peer flag is never raised: the wait runs out after the limit given to the launch, the kernel
    records status 105 and returns through its normal teardown, and the next launch on the same context works."""
    from sllm_b200 import ops
    from sllm_b200.ops import fused_decode as fd
    from sllm_b200.ops import reference as ref
    from sllm_b200.ops.core import LinearWeight
    from sllm_b200.parallel.tp import CommDesc
    dev = torch.device("cuda")
    rows, d, k, bn = 4, 256, 256, 16
    g = torch.Generator().manual_seed(0)
    lw = LinearWeight.from_dense((torch.randn(d, k, generator=g) * 0.03).bfloat16(), "fp8").to(dev)
    xq, xs_t = ref.quant_fp8_1x128((torch.randn(rows, k, generator=g)).bfloat16())
    xs = torch.zeros((k // 128, bn)); xs[:, :rows] = xs_t
    xq, xs = xq.to(dev), xs.to(dev)
    h = torch.zeros((rows, d), dtype=torch.bfloat16, device=dev)
    q = torch.zeros((rows, d), dtype=torch.uint8, device=dev)
    s = torch.zeros((d // 128, bn), dtype=torch.float32, device=dev)
    ssq = torch.zeros((d // 128, bn), dtype=torch.float32, device=dev)
    ph = fd.phase(fd.RESID_QUANT, lw.w, lw.scale_t, xq, xs, n=d, k=k, y=h, ldy=d, residual=h, q_out=q, s_out=s, ssq_out=ssq,
                  ld_s_out=bn)
    # a two-rank communicator whose "peer" is this GPU's own memory and never answers
    recv = torch.zeros(2 * 2 * 32 * d, dtype=torch.bfloat16, device=dev)
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    epoch = torch.zeros(16, dtype=torch.int32, device=dev)
    comm = CommDesc()
    comm.world, comm.rank, comm.cap_elems, comm.max_tiles = 2, 0, 32 * d, d // 128
    for r in range(2):
        comm.recv[r], comm.flags[r] = recv.data_ptr(), flags.data_ptr()
    comm.epoch = epoch.data_ptr()
    assert ops.device_status(dev) == 0
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    fd.launch([ph], rows, dev, comm=comm, impl="persistent", wait_limit_cycles=4_000_000)     # ~2 ms
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 2000.0                  # it gave up after the limit, not after the library default
    assert ops.device_status(dev) == 105                 # timeout waiting for a peer flag (reading clears the word)
    fd.reset_state(dev)
    y = torch.zeros((rows, d), dtype=torch.bfloat16, device=dev)
    ok = fd.phase(fd.PLAIN, lw.w, lw.scale_t, xq, xs, n=d, k=k, y=y, ldy=d)
    fd.launch([ok], rows, dev, impl="persistent")
    want = fd.ref_plain(lw.w, lw.scale_t, xq, xs, rows)
    assert ((y.float().cpu() - want).norm() / want.norm()).item() < 6e-3
    assert ops.device_status(dev) == 0


@pytest.mark.gpu
def test_kernel_trace_tool_output_schema(capsys):
    """The tracing tool's JSON form is stable: schema id, column names, one row per tile / phase, stamps that increase
    along a row where taken."""
    import json
    from sllm_b200.utils import kernel_trace
    assert kernel_trace.main(["--op", "fused-decode", "--batch", "8", "--json"]) == 0
    doc = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert doc["schema"] == "sllm-kernel-trace-v1" and doc["op"] == "fused-decode" and doc["cold_us"] > 0
    assert len(doc["rows"]) == 4 and all(len(r) == len(doc["columns"]) for r in doc["rows"])
    col = {n: i for i, n in enumerate(doc["columns"])}
    for r in doc["rows"]:
        assert r[col["input_visible.first"]] <= r[col["first_accumulator.first"]] <= r[col["barrier_arrival.last"]]
    # each phase starts after the previous one's last barrier arrival
    for a, b in zip(doc["rows"], doc["rows"][1:]):
        assert b[col["input_visible.first"]] >= a[col["barrier_arrival.last"]]


def test_fail_closed_mode_never_computes_on_cpu():
    """With fail-closed mode on, an op handed a CPU tensor raises instead of computing its PyTorch oracle."""
    import torch
    from sllm_b200 import ops
    from sllm_b200.ops import _lib
    x = torch.randn(2, 128)
    w = torch.ones(128)
    assert ops.rmsnorm(x, w, 1e-5).shape == (2, 128)            # the CPU oracle path, as the CPU tests use it
    _lib.set_fail_closed(True)
    try:
        for call in (lambda: ops.rmsnorm(x, w, 1e-5), lambda: ops.argmax(torch.randn(2, 16)),
                     lambda: ops.embedding(torch.randn(4, 8), torch.tensor([1, 2], dtype=torch.int32))):
            try:
                call()
            except _lib.KernelError as exc:
                assert "fail-closed" in str(exc)
            else:
                raise AssertionError("a CPU tensor was computed in fail-closed mode")
    finally:
        _lib.set_fail_closed(False)
    assert ops.rmsnorm(x, w, 1e-5).shape == (2, 128)


def test_quarantine_accounting_and_release():
    """A device failure quarantines the engine: every entry point refuses, the backend stops accepting, the report
    says why; memory is freed only when the device work is known to be complete, otherwise it is parked."""
    import pytest
    import torch
    from sllm_b200.engine import engine as E
    from sllm_b200.models import config as MC
    eng = E.build_engine(MC.tiny_llama(), "cpu", seed=1, num_pages=16, max_batch=2, use_cuda_graphs=False)
    acc = eng.accounting()
    assert acc["weights"] > 0 and acc["kv_pages"] == eng.cache.values.numel() * eng.cache.values.element_size()
    assert acc["captured_graphs"] == 0 and acc["pinned_host"] > 0
    out = eng.generate([[1, 2, 3]], 3)
    eng._enter_quarantine("a bounded device wait gave up (status 105)", 105)
    for call in (lambda: eng.new_sequence([1, 2]), lambda: eng.generate([[1, 2, 3]], 2)):
        with pytest.raises(E.EngineQuarantined):
            call()
    rep = eng.shutdown_report()
    assert rep["quarantine"]["device_status"] == 105 and rep["quarantine"]["work_completed"] and rep["steps"] >= 2
    assert rep["kv_pool"] is not None and "fallbacks" in rep
    freed = eng.release()
    assert freed["freed_bytes"] == acc["kv_pages"] and freed["parked_bytes"] == 0 and eng.cache.values.numel() == 0
    # work that cannot be proven complete: nothing is freed, the buffers stay referenced
    e2 = E.build_engine(MC.tiny_llama(), "cpu", seed=1, num_pages=16, max_batch=2, use_cuda_graphs=False)
    e2._enter_quarantine("synchronize failed", 0)
    e2.quarantine["work_completed"] = False
    n = len(E._PARKED)
    r2 = e2.release()
    assert r2["freed_bytes"] == 0 and r2["parked_bytes"] > 0 and len(E._PARKED) == n + 1 and e2.cache.values.numel() > 0
    assert out and len(out[0]) == 3


def test_fake_kernel_library_scripts_launch_failures():
    """The programmable fake of the kernel library: calls are recorded, scripted status codes come back as KernelError
    naming the status, successful launches are counted, and an engine step that hits a rejected launch fails without
    committing anything, so the same sequence decodes again afterwards."""
    import pytest
    import torch
    from sllm_b200 import ops
    from sllm_b200.engine.engine import build_engine
    from sllm_b200.models import config as MC
    from sllm_b200.ops import _lib
    x, w = torch.randn(3, 256), torch.ones(256)
    want = ops.rmsnorm(x, w, 1e-5)
    fake = _lib.FakeKernelLibrary({"sllm_rmsnorm": [0, 3]})
    _lib.install_fake(fake)
    try:
        n0 = _lib.LAUNCH_COUNT[0]
        y = ops.rmsnorm(x, w, 1e-5)                                   # "launched": allocated, not computed
        assert y.shape == want.shape and fake.count("sllm_rmsnorm") == 1 and _lib.LAUNCH_COUNT[0] == n0 + 1
        name, args = fake.calls[0]
        assert name == "sllm_rmsnorm" and args[0].value == x.data_ptr()
        with pytest.raises(_lib.KernelError) as ei:
            ops.rmsnorm(x, w, 1e-5)
        assert _lib.STATUS_NAMES.get(3, "3") in str(ei.value) and _lib.LAUNCH_COUNT[0] == n0 + 1
        with pytest.raises(AttributeError):
            fake.sllm_no_such_entry_point
    finally:
        _lib.install_fake(None)
    assert torch.equal(ops.rmsnorm(x, w, 1e-5), want)                  # the real (CPU oracle) path is back
    # an engine step under a fake that rejects the 5th GEMM launch
    eng = build_engine(MC.tiny_llama(), "cpu", seed=1, num_pages=16, max_batch=2, use_cuda_graphs=False)
    s = eng.new_sequence([3, 4, 5, 6])
    first = eng.prefill([s])[0]
    s.tokens.append(first)
    computed = s.num_computed
    fake = _lib.FakeKernelLibrary({"sllm_gemm": [0, 0, 0, 0, 9]})
    _lib.install_fake(fake)
    try:
        with pytest.raises(_lib.KernelError):
            eng.decode([s])
        assert fake.count("sllm_gemm") == 5
    finally:
        _lib.install_fake(None)
    assert s.num_computed == computed and eng.cache.pool.length(s.seq_id) == computed      # nothing was committed
    tok = eng.decode([s])[0]
    ref_eng = build_engine(MC.tiny_llama(), "cpu", seed=1, num_pages=16, max_batch=2, use_cuda_graphs=False)
    r = ref_eng.new_sequence([3, 4, 5, 6])
    r.tokens.append(ref_eng.prefill([r])[0])
    assert tok == ref_eng.decode([r])[0]

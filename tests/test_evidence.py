"""Evidence runners: report schema, fail-closed behaviour without a GPU, the dispatch audit ring; on a GPU every op of
the registry produces a passing report."""
import json

import pytest
import torch

from sllm_b200 import evidence as EV
from sllm_b200.ops import _lib


def test_reports_without_a_gpu_state_why_and_compute_nothing(capsys):
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from sllm_b200.evidence.runner import main
    assert main(["--all"]) == 0
    lines = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines()]
    assert {r["op"] for r in lines} == set(EV.OPS) and all(not r["executed"] and "CUDA" in r["unavailable"] for r in lines)
    for r in lines:
        EV.validate_report(r)
    assert main([]) == 2 and main(["--op", "rmsnorm", "--all"]) == 2
    with pytest.raises(ValueError):
        EV.validate_report({"schema": EV.SCHEMA, "op": "x", "executed": True})
    with pytest.raises(ValueError):
        EV.validate_report({"schema": "other", "op": "x", "executed": False, "unavailable": "y"})


def test_dispatch_audit_ring_is_bounded_and_off_by_default():
    _lib.audit(False)
    _lib.dispatch_records(clear=True)
    _lib.record_dispatch("linear", "gemm_tcgen05_kernel", m=1)
    assert _lib.dispatch_records() == []
    _lib.audit(True)
    try:
        for i in range(300):
            _lib.record_dispatch("linear", "gemm_tcgen05_kernel", fallback_used=(i == 299), m=i)
        recs = _lib.dispatch_records()
        assert len(recs) == 256 and recs[-1]["m"] == 299 and recs[-1]["fallback_used"] and recs[0]["m"] == 44
        assert recs[-1]["seq"] - recs[0]["seq"] == 255
        assert _lib.dispatch_records(clear=True) and _lib.dispatch_records() == []
    finally:
        _lib.audit(False)


@pytest.mark.gpu
@pytest.mark.parametrize("op", sorted(EV.OPS))
def test_every_runner_passes_on_the_gpu(op):
    rep = EV.run_op(op, "small")
    EV.validate_report(rep)
    assert rep["executed"] and rep["correctness"]["passed"], rep["correctness"]
    assert rep["timing"]["median_us"] > 0 and rep["device"]["device_status"] == 0
    if op.startswith("gemm-") or op == "paged-attention-fp8":
        assert rep["dispatch"] and not any(d["fallback_used"] for d in rep["dispatch"])


def test_roundtrip_reaper_and_circuit_breaker(tmp_path):
    """The model-free round trip: a child that overstays is reaped by pid, consecutive failures open the breaker, an
    open breaker attempts nothing, the cooldown lets one trial through and a success closes it."""
    import sys
    from sllm_b200.evidence import roundtrip as RT
    now = [1000.0]
    kw = dict(state_dir=str(tmp_path), threshold=2, cooldown=60.0, clock=lambda: now[0])
    ok_cmd = [sys.executable, "-c", 'print(\'{"ok": true, "checks": {}}\')']
    bad_cmd = [sys.executable, "-c", 'import sys; print(\'{"ok": false}\'); sys.exit(1)']
    hang_cmd = [sys.executable, "-c", "import time; time.sleep(60)"]
    r = RT.roundtrip(cmd=ok_cmd, **kw)
    assert r["ok"] and r["circuit"] == "closed" and r["attempted"] and not r["reaped"]
    r = RT.roundtrip(cmd=hang_cmd, timeout=0.5, **kw)
    assert not r["ok"] and r["reaped"] and r["consecutive_failures"] == 1 and r["circuit"] == "closed"
    r = RT.roundtrip(cmd=bad_cmd, **kw)
    assert not r["ok"] and r["consecutive_failures"] == 2 and r["circuit"] == "open"
    r = RT.roundtrip(cmd=ok_cmd, **kw)                                   # open: not even attempted
    assert r["circuit"] == "open" and not r["attempted"]
    now[0] += 61
    r = RT.roundtrip(cmd=bad_cmd, **kw)                                  # half-open trial fails: open again, clock restarts
    assert r["attempted"] and r["circuit"] == "open"
    assert not RT.roundtrip(cmd=ok_cmd, **kw)["attempted"]
    now[0] += 61
    r = RT.roundtrip(cmd=ok_cmd, **kw)
    assert r["ok"] and r["circuit"] == "closed" and r["consecutive_failures"] == 0
    # "no GPU" neither trips nor resets the breaker
    none_cmd = [sys.executable, "-c", 'print(\'{"ok": false, "unavailable": "no CUDA device"}\')']
    RT.roundtrip(cmd=bad_cmd, **kw)
    r = RT.roundtrip(cmd=none_cmd, **kw)
    assert r["consecutive_failures"] == 1 and r["attempted"]
    if not torch.cuda.is_available():
        assert RT.main(["--state-dir", str(tmp_path / "real")]) == 0      # the real child: unavailable here, exit 0


@pytest.mark.gpu
def test_roundtrip_on_the_gpu(tmp_path):
    from sllm_b200.evidence import roundtrip as RT
    r = RT.roundtrip(state_dir=str(tmp_path), timeout=240.0)
    assert r["ok"] and r["device_status"] == 0 and r["circuit"] == "closed", r
    assert set(r["checks"]) == {"gemm_bf16", "gemm_fp8", "rmsnorm", "gated_act", "argmax", "paged_attention"}


def test_accuracy_runner_orders_the_formats_on_the_cpu():
    """KL(bf16 || candidate) over shared seeded weights: identical configurations give zero, FP8 moves the distribution
    less than 4-bit weights, and 4-bit activations add to the 4-bit weights' divergence."""
    from sllm_b200.evidence import accuracy as ACC
    same = ACC.compare("bf16", "bf16", device="cpu", prompts=3, prompt_len=12)
    assert same["kl_mean"] == 0.0 and same["top1_agreement"] == 1.0
    fp8 = ACC.compare("bf16", "fp8", device="cpu", prompts=3, prompt_len=12)
    w4 = ACC.compare("bf16", "nvfp4", device="cpu", prompts=3, prompt_len=12)
    w4a4 = ACC.compare("bf16", "nvfp4", act4=True, device="cpu", prompts=3, prompt_len=12)
    assert 0.0 < fp8["kl_mean"] < w4["kl_mean"] < w4a4["kl_mean"] and w4a4["finite"]
    assert w4a4["candidate"] == "nvfp4+act4" and w4a4["schema"] == "sllm-accuracy-v1"
    with pytest.raises(ValueError):
        ACC.compare("bf16", "fp8", act4=True, device="cpu")


@pytest.mark.gpu
def test_accuracy_runner_on_the_gpu():
    from sllm_b200.evidence import accuracy as ACC
    rep = ACC.compare("bf16", "nvfp4", act4=True, device="cuda", prompts=4, prompt_len=16)
    cpu = ACC.compare("bf16", "nvfp4", act4=True, device="cpu", prompts=4, prompt_len=16)
    assert rep["finite"] and 0.0 < rep["kl_mean"] < 4 * cpu["kl_mean"] + 1e-3

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

"""Leader/follower protocol over gloo with two CPU ranks."""
import os
import subprocess
import sys


def test_leader_follower_cpu():
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29833", os.path.join(here, "dist_engine_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert proc.returncode == 0 and "DIST_ENGINE_OK" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-3000:]


def _run_failure_case(case: str, port: int):
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, SLLM_TEST_FAIL=case)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(here, "dist_failure_worker.py")]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)


def test_follower_failure_reaches_the_leader_on_the_host():
    """A follower that raises while replaying a step posts the error and leaves; the leader raises before its next
    launch instead of waiting for the dead rank."""
    proc = _run_failure_case("follower_raises", 29835)
    out = proc.stdout
    assert "FOLLOWER_REPORTED_AND_LEFT" in out and "LEADER_SAW_FOLLOWER_FAILURE" in out and "NO_FAILURE_SEEN" not in out, \
        out[-2000:] + proc.stderr[-3000:]


def test_follower_notices_a_leader_that_went_away():
    proc = _run_failure_case("leader_stops", 29836)
    out = proc.stdout
    assert "LEADER_EXITS_WITHOUT_STOP" in out and "FOLLOWER_SAW_LEADER_LOSS" in out, out[-2000:] + proc.stderr[-3000:]

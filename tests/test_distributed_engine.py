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

"""Tensor-parallel paths on 2+ GPUs: fused GEMM+all-reduce vs the NCCL baseline vs fp32 maths."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29611 + world), os.path.join(here, "tp_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and "TP_WORKER_OK" in proc.stdout, proc.stdout[-3000:] + proc.stderr[-3000:]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29711 + world), os.path.join(here, "ep_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and "EP_WORKER_OK" in proc.stdout, proc.stdout[-3000:] + proc.stderr[-3000:]

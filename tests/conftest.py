import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")
    config.addinivalue_line("markers", "multigpu: needs more than one GPU")


@pytest.fixture(scope="session", autouse=True)
def _native_libs():
    """Build the host library (and the kernel library when nvcc is present) once per session."""
    from sllm_b200 import build
    build.build_host()
    try:
        build.build_kernels()
    except RuntimeError:
        pass
    yield


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)

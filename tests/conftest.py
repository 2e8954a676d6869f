import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "vllm-xpu-kernels_b200")
for p in (ROOT, PKG_DIR):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Arrays of tests/golden/<name>.npz as torch tensors (bf16 / fp8 were
    stored as raw integers and are viewed back by key convention)."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return {k: torch.from_numpy(z[k]) if z[k].ndim else z[k].item() for k in z.files}


def as_bf16(t):
    return t.view(torch.bfloat16)


@pytest.fixture(scope="session")
def ops():
    """torch.ops namespaces with the CUDA operators registered."""
    import vllm_xpu_kernels._C  # noqa: F401
    import vllm_xpu_kernels._moe_C  # noqa: F401
    import vllm_xpu_kernels._xpu_C  # noqa: F401
    return torch.ops


@pytest.fixture(autouse=True)
def _check_device_status(request):
    yield
    if "gpu" in request.keywords and torch.cuda.is_available():
        import vllm_xpu_kernels._xpu_C  # noqa: F401
        st = torch.ops._xpu_C.b200_device_status()
        assert st == 0, f"a bounded device-side wait gave up (status {st})"

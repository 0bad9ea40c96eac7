import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")
    # The CUDA library is built in-tree and kept out of version control: build it when a fresh checkout lacks it
    # (nvcc cross-compiles for sm_100a without a GPU).
    from t0_gpu_b200 import _lib, build as lib_build

    if not os.path.exists(_lib.LIB_PATH):
        lib_build.build()


def _has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this environment")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def rt():
    """One runtime per test process, like the reference's shared `OnceLock<GpuRuntime>`
    (src/t0/tile_ir.rs:3483-3497)."""
    import t0_gpu_b200 as t

    r = t.GpuRuntime()
    yield r
    r.close()

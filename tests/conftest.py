"""Shared pytest set-up: the `gpu` marker, import paths, and helpers that load
the native libraries (built by ``__graft_entry__.build()`` / ``build.py``)."""
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
PKG_DIR = ROOT / "vllm-xpu-kernels_b200"
for p in (str(ROOT), str(PKG_DIR)):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def native():
    """The Python surface with the native op libraries loaded (fails loudly if
    they were not built)."""
    import vllm_xpu_kernels.fused_moe_interface as fmi
    assert fmi.FUSEDMOE_AVAILABLE, f"native libraries missing: {fmi.FUSEDMOE_UNAVAILABLE_REASON}"
    return fmi


def load_golden(name):
    return torch.load(GOLDEN / name, weights_only=False)

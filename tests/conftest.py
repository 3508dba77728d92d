import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a) and the built kernel library")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _no_index_outside_its_range(request):
    """When the whole suite runs on the checked build of the kernels (``BSPEC_BOUNDS=1 python -m pytest tests -m
    gpu``), every GPU test also fails if a kernel recorded an index outside its range while it ran.  Nothing to do
    on the ordinary build."""
    yield
    if os.environ.get("BSPEC_BOUNDS", "0") != "1" or "gpu" not in request.keywords:
        return
    if request.node.name.startswith("test_checked_build") or request.node.name.startswith("test_ordinary_build"):
        return
    from batchspec_b200.kernels import ops
    found = ops.bounds_reports()
    assert not found, found

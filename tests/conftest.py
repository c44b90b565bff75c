"""Test configuration: the ``gpu`` marker and shared fixtures.

``-m "not gpu"`` tests run anywhere; ``-m gpu`` tests need a B200 and are skipped (not
failed) where no CUDA device is visible.  Model folders are written into temporary folders.
"""
import os
import sys
from pathlib import Path

import pytest
import torch

# every buffer the engine allocates without a value starts as NaN in the tests: a kernel that reads memory
# nobody wrote then shows as NaN instead of depending on what the memory held before
os.environ.setdefault("TESSWEAVE_POISON_BUFFERS", "1")

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device visible")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder of the tiny model with weights stored in bf16 (exact in both run types)."""
    from helpers import make_folder
    tmp = tmp_path_factory.mktemp("models")
    return {name: make_folder(tmp, name) for name in ("A", "B", "C")}

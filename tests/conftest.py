import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def reference_dir():
    """The reference checkout (for tests that read its plan files): $ARK_REFERENCE_DIR, else a `reference`
    directory beside this repository; None when there is none."""
    for d in (os.environ.get("ARK_REFERENCE_DIR"), os.path.join(os.path.dirname(ROOT), "reference")):
        if d and os.path.isdir(os.path.join(d, "examples", "tutorial")):
            return d
    return None


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)

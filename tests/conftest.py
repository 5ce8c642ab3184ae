import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _restore_default_dtype():
    before = torch.get_default_dtype()
    yield
    torch.set_default_dtype(before)


def reference_library():
    """The unmodified upstream package (installed under baseline/_ref), or None."""
    for root in (os.environ.get("PSGD_REFERENCE_ROOT"), os.path.join(ROOT, "baseline", "_ref")):
        if root and os.path.isdir(os.path.join(root, "powersgd")):
            if root not in sys.path:
                sys.path.append(root)
            try:
                import powersgd  # noqa: F401

                return powersgd
            except Exception:
                return None
    return None

"""pytest configuration: markers and import paths shared by every test."""

import os
import sys

os.environ.setdefault("TRI_B200_CHECK", "1")  # make a timed-out tensor-core wait fail the test loudly

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_sessionstart(session):
    """Build the CUDA library in-tree if it is missing or older than its sources (nvcc only, no GPU needed)."""
    from geometric_nn_ops_b200.build import build_library
    try:
        build_library()
    except Exception as exc:  # a box without nvcc still runs with a prebuilt library
        lib = os.path.join(ROOT, "geometric_nn_ops_b200", "libtri_b200.so")
        if not os.path.exists(lib):
            raise RuntimeError(f"libtri_b200.so is missing and could not be built: {exc}") from exc

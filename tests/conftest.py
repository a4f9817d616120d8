import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def lib_built():
    """Build the CUDA library if nvcc is here; GPU boxes use the prebuilt file."""
    from megakernels_b200 import build
    import shutil
    if shutil.which("nvcc"):
        build.build()
    assert os.path.exists(build.LIB), "libmk_b200.so missing"
    return build.LIB

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_PARENT = os.path.join(ROOT, "flash-attention_b200")
for p in (ROOT, PKG_PARENT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")
    # The C-ABI library must exist for every test that touches the package; build it once when a
    # fresh checkout has not been built yet (nvcc cross-compiles without a GPU).
    lib = os.path.join(PKG_PARENT, "flash_attn_b200", "libfa_b200.so")
    if not os.path.exists(lib):
        sys.path.insert(0, PKG_PARENT)
        import build as fa_build
        fa_build.build()


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")

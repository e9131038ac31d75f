import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")

# The GEMM switches to its 512-column tile only for deep reductions (K >= 8192 by default); lower the threshold
# so that the test sizes reach that kernel too (read once by the library, at its first GEMM).
os.environ.setdefault("BFB_GEMM_WIDE_K", "1024")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_ops():
    return dict(np.load(os.path.join(GOLDEN, "ops.npz")))


@pytest.fixture(scope="session")
def golden_c1_default():
    return dict(np.load(os.path.join(GOLDEN, "c1_default.npz")))


@pytest.fixture(scope="session")
def golden_c1_normal():
    return dict(np.load(os.path.join(GOLDEN, "c1_normal.npz")))


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU backend (oracle/_ref), when the prebuilt library is present."""
    from oracle import ref_lib
    if not ref_lib.available():
        pytest.skip("oracle/_ref/libbf_ref.so not built")
    return ref_lib


@pytest.fixture(scope="session")
def bfb():
    import blackforge_b200
    blackforge_b200.lib()  # raises if the CUDA library is missing: no fallback
    return blackforge_b200


@pytest.fixture(scope="session")
def gpu(bfb):
    if not bfb.has_gpu():
        pytest.fail("a test marked gpu is running without a usable CUDA device")
    return bfb

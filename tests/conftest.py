import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "tests", ROOT / "tests" / "golden"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def built_lib():
    """Builds (if stale) and loads the CUDA library; GPU tests fail loudly without it."""
    from llminfer_b200 import build
    build.build_kernels()
    from llminfer_b200 import binding
    return binding.lib()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = ROOT / "tests" / "golden" / "ref_cuda_bf16.npz"
    if not path.exists():
        pytest.skip("golden file not generated yet")
    return np.load(path)

import sys
from pathlib import Path

import pytest

# torch first: importing it after the reference engine's shared library (its OpenMP and BLAS pieces) has been loaded
# into the process crashes inside torch's own start-up
try:
    import torch  # noqa: F401
except ImportError:
    pass

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "oracle", ROOT / "tests", ROOT / "tests" / "golden"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle_lib import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(ROOT / "tests" / "golden" / "reference_cpu_engine.npz")


@pytest.fixture(scope="session")
def reference():
    """The reference's own CPU engine, where oracle/_ref has been built; tests that need it skip otherwise."""
    from oracle_lib import Reference
    if not Reference.available():
        pytest.skip("oracle/_ref not built (needs a NeoML checkout: make -C oracle ref)")
    ref = Reference()
    yield ref
    ref.close()

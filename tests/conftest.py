import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Byte fixtures produced by the reference's own code (see tests/golden/make_golden.py)."""
    with np.load(os.path.join(ROOT, "tests", "golden", "ggml_path_golden.npz")) as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def port():
    from oracle import oracle as O
    return O.port()


@pytest.fixture(scope="session")
def ref():
    from oracle import oracle as O
    if not O.ref_available():
        pytest.skip("oracle/_ref not built (needs a reference checkout at build time)")
    return O.ref()

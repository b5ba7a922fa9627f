import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as orc
    return orc.Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own code (oracle/_ref); built when a reference checkout is present, else the test is skipped."""
    from oracle import oracle as orc
    try:
        path = orc.build_reference()
    except Exception:  # a checkout that does not build is reported by test_oracle_ref.py, not here
        path = None
    if not path:
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    return orc.Reference(path)


@pytest.fixture(scope="session")
def golden():
    import json
    import numpy as np
    g = os.path.join(ROOT, "tests", "golden")

    class G:
        def npz(self, name):
            return np.load(os.path.join(g, name + ".npz"))

        def json(self, name):
            with open(os.path.join(g, name + ".json")) as f:
                return json.load(f)
    return G()

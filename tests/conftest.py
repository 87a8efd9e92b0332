import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    """The plain-C CPU oracle, built on demand (test infrastructure, never the product path)."""
    from oracle import build as oracle_build
    oracle_build.build_oracle()
    from oracle.oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    gdir = os.path.join(ROOT, "tests", "golden")
    return {name: np.load(os.path.join(gdir, "reference_%s.npz" % name)) for name in ("ops", "logits", "optimizer", "ranking")}


@pytest.fixture(autouse=True)
def _no_abandoned_copy_waits(request):
    """After every GPU test: no kernel of the library gave up waiting for a bulk copy."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import torch
        if torch.cuda.is_available():
            from smore_b200 import _lib
            assert _lib.async_status() == 0, "a bulk-copy wait ran out inside a kernel"

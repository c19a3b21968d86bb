import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "graph-compiler_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    import json

    import numpy as np

    g = os.path.join(ROOT, "tests", "golden")
    with open(os.path.join(g, "benchgc_golden.json")) as f:
        meta = json.load(f)
    arrays = np.load(os.path.join(g, "benchgc_golden.npz"))
    return meta, arrays

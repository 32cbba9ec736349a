import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


class Golden:
    """Read-only view of one of the .npz files under tests/golden/."""

    def __init__(self, fname):
        self._z = np.load(os.path.join(ROOT, "tests", "golden", fname), allow_pickle=False)
        self.meta = json.loads(str(self._z["__meta__"]))

    def case(self, name):
        prefix = name + "/"
        return {k[len(prefix):]: self._z[k] for k in self._z.files if k.startswith(prefix)}

    def names(self, kind=None):
        return [n for n, m in self.meta.items()
                if not n.startswith("__") and (kind is None or m.get("kind") == kind)]


@pytest.fixture(scope="session")
def perturbed_golden():
    return Golden("perturbed_golden.npz")


@pytest.fixture(scope="session")
def binary_golden():
    return Golden("binary_golden.npz")

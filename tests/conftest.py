import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Golden:
    """Committed input/output vectors produced by the reference's own torch functions."""

    def __init__(self):
        self._z = np.load(os.path.join(ROOT, "tests", "golden", "reference_vectors.npz"))

    def case(self, name, bf16=()):
        out = {}
        for key in self._z.files:
            c, k = key.split("/")
            if c != name:
                continue
            t = torch.from_numpy(self._z[key].copy())
            if k in bf16:
                t = t.view(torch.int16).view(torch.bfloat16)
            out[k] = t
        assert out, name
        return out


@pytest.fixture(scope="session")
def golden():
    return Golden()

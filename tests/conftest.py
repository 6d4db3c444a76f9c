import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


GOLDEN_CASES = ["blobs_n600_d5_k4", "blobs_n2000_d32_k8", "empty_n500_d3_k6", "blobs_n1500_d7_k17",
                # shapes the tcgen05 kernels serve (resident and streamed centroid table)
                "blobs_n3000_d64_k100", "blobs_n3600_d128_k300"]


@pytest.fixture(scope="session")
def built_lib():
    """Path of the in-tree shared library (built on demand, never a CPU stand-in)."""
    from h2o4gpu_b200 import build
    return build.build()

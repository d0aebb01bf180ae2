import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")
PRECS = ["fp32", "fp16", "bf16", "int8", "int4", "int2"]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def spg():
    """The product package with its C library loaded (built here if missing)."""
    import spingalett_b200
    if not os.path.exists(spingalett_b200.LIB_PATH):
        from spingalett_b200 import build
        build.build()
    spingalett_b200.lib().spingalett_set_verbose(False)
    return spingalett_b200


@pytest.fixture(scope="session")
def oracle():
    import oracle as o
    if not os.path.exists(o.ORACLE_SO):
        o.build_oracle()
    return o


@pytest.fixture(scope="session")
def has_gpu(spg):
    return spg.lib().spingalett_get_device_count() > 0


@pytest.fixture(autouse=True)
def _clear_error(spg):
    spg.lib().spingalett_clear_error()
    yield
    spg.lib().spingalett_clear_error()


def golden(name):
    return os.path.join(GOLDEN, name)


def ulp_diff(a, b):
    """Largest distance in units in the last place between two float32 arrays."""
    a = np.ascontiguousarray(a, np.float32).view(np.int32).astype(np.int64)
    b = np.ascontiguousarray(b, np.float32).view(np.int32).astype(np.int64)
    a = np.where(a < 0, -(a & 0x7FFFFFFF), a)
    b = np.where(b < 0, -(b & 0x7FFFFFFF), b)
    return int(np.abs(a - b).max()) if a.size else 0

"""Test configuration: the ``gpu`` marker, library/oracle fixtures and seeded-input helpers.

CPU tests (``-m "not gpu"``) cover the oracle against golden vectors and independent implementations,
the host logic and the C-ABI surface.  GPU tests (``-m gpu``) are the parity tests proper: they call the
CUDA path through the C ABI and compare with the oracle on the same seeded inputs.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")
REL_TOL = 1e-2  # max|err| <= 1e-2 * max|ref|, the acceptance bound of the benchmark configurations


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def O():
    from oracle import oracle

    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def native():
    """Builds (if needed) and loads libb200gemm.so; fails loudly when that is impossible."""
    from gcnasm_b200 import build

    build.build_library()
    from gcnasm_b200 import _lib

    return _lib.lib()


@pytest.fixture(scope="session")
def api(native):
    from gcnasm_b200 import api

    return api


def assert_close(O, got, ref, what=""):
    err, mref = O.max_err(np.asarray(ref, np.float32), np.asarray(got, np.float32))
    assert err <= REL_TOL * mref, f"{what}: max|err|={err:.4g} exceeds 1e-2*max|ref|={REL_TOL * mref:.4g}"
    return err, mref

"""Shared pytest setup: import paths, the `gpu` marker, and GPU fixtures.

`-m "not gpu"` runs the oracle, the host logic and the C-ABI load/validation
checks on CPU.  `-m gpu` tests are the parity tests proper: they call the CUDA
library through its C ABI and compare with the oracle.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "ullm-project_b200"), os.path.join(ROOT, "oracle"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device; run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "quant_linear_v1.npz"))


@pytest.fixture(scope="session")
def gpu():
    """(context, queue) on cuda:0.  Fails — never skips — when the CUDA library
    or device is missing, so that a GPU run cannot pass on a fallback."""
    import ullm_cuda as U

    probe = U.backend_probe()
    assert probe.available, f"CUDA backend unavailable on a GPU test run: {probe.diagnostic}"
    ctx = U.Context(0)
    q = ctx.queue()
    yield ctx, q
    q.close()

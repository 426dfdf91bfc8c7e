"""Shared fixtures.  Tests that need a B200 carry ``@pytest.mark.gpu``; the
rest run on CPU only.  Following the reference's gate
(scripts/test.sh:10-18, crates/metal/src/tests.rs:13-25) a missing device is a
loud skip, and a failure when ``TUCKMILL_REQUIRE_CUDA=1``."""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA sm_100 device (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def ctx():
    from tuckmill_b200 import cuda
    if cuda.available() == 0:
        msg = "no sm_100 CUDA device: GPU parity tests did not run"
        if os.environ.get("TUCKMILL_REQUIRE_CUDA") == "1":
            pytest.fail(msg)
        print("\n*** SKIP: " + msg + " ***")
        pytest.skip(msg)
    c = cuda.CudaContext(0)
    yield c
    c.close()


def rel_err(gpu, cpu):
    """The reference's device-test tolerance rule: max|gpu-cpu| / max(1, max|cpu|)
    (crates/metal/src/tests.rs:367-381)."""
    import numpy as np
    gpu = np.asarray(gpu, dtype=np.float64)
    cpu = np.asarray(cpu, dtype=np.float64)
    return float(np.max(np.abs(gpu - cpu)) / max(1.0, float(np.max(np.abs(cpu)))))

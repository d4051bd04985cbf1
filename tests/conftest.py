import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Parity bar, stated once: both figures are measured on fp32 outputs against the
# CPU checker fed the same (cast-then-upcast) inputs.
REL_L2_TOL = 1e-3
MAX_ABS_TOL = 1e-3   # as a fraction of the largest column mean


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def golden():
    """(manifest cases, arrays) of outputs produced by the reference's naive_colsum."""
    from flash_colsum_b200.inputs import Workload
    gdir = os.path.join(ROOT, "tests", "golden")
    with open(os.path.join(gdir, "naive_colsum_golden.json")) as f:
        manifest = json.load(f)
    arrays = np.load(os.path.join(gdir, "naive_colsum_golden.npz"))
    cases = []
    for c in manifest["cases"]:
        sha = c.pop("sha256")
        cases.append((Workload(**c), sha))
    return cases, arrays

"""Shared pytest scaffolding: markers, the (u, gs) sweep, seeded RNG, helpers."""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

U_VALUES = (2, 3, 4)
GS_VALUES = (2, 4, 8)
CONFIGS = [(u, gs) for u in U_VALUES for gs in GS_VALUES]

# Output tolerances of the decode path against the float64 oracle fed the same
# bf16-rounded inputs.  Kernels return bf16; both metrics are taken against the
# oracle result rounded to bf16 (the output's storage precision):
#   max_abs_rel = max|got - ref| / max|ref|   <= 2^-7
#   rel_fro     = ||got - ref|| / ||ref||     <= 1e-3
MAX_ABS_REL_TOL = 2.0 ** -7
REL_FRO_TOL = 1e-3
# The same comparison before the final bf16 rounding (float32 outputs of the C ABI).
F32_REL_FRO_TOL = 2e-5


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture
def rng():
    return np.random.default_rng(11)


@pytest.fixture(params=CONFIGS, ids=[f"u{u}_gs{gs}" for (u, gs) in CONFIGS])
def cfg(request):
    return request.param


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "msaq_golden.npz")
    with np.load(path) as z:
        return {k: z[k] for k in z.files}

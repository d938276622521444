"""pytest configuration: the `gpu` marker and shared fixture loaders."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def ops_golden():
    """Op-level vectors produced by the reference's CPU code (tests/golden/make_golden_ops.py)."""
    with np.load(ROOT / "tests" / "golden" / "ops_golden.npz") as z:
        return {k: z[k] for k in z.files}

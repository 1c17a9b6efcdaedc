"""Shared fixtures: markers, the repository root on sys.path, golden-vector loaders."""
import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    class G:
        meta = json.loads((GOLDEN / "golden_meta.json").read_text())

        @staticmethod
        def load(name):
            return np.load(GOLDEN / f"{name}.npz")
    return G

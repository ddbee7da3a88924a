from __future__ import annotations

import os
import sys
import tempfile
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# keep schedule caches and probe logs of the tests out of the user's home directory
os.environ.setdefault("AUTOSAGE_CACHE_DIR", tempfile.mkdtemp(prefix="autosage-test-cache-"))
os.environ.setdefault("AUTOSAGE_LOG_PROBES", "0")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "cuda: alias used by the reference's tests")


@pytest.fixture(scope="session")
def native_library():
    """Path of libautosage_b200.so, built on demand (nvcc cross-compiles without a GPU)."""
    from autosage_b200 import build as builder

    return builder.build()


@pytest.fixture(scope="session")
def golden():
    import json

    import numpy as np

    folder = ROOT / "tests" / "golden"
    vectors = np.load(folder / "reference_vectors.npz")
    keys = json.loads((folder / "reference_keys.json").read_text(encoding="utf-8"))
    return vectors, keys


@pytest.fixture()
def isolated_cache(tmp_path, monkeypatch):
    monkeypatch.setenv("AUTOSAGE_CACHE_DIR", str(tmp_path))
    return tmp_path

"""Shared test plumbing: the `gpu` marker, the oracle handles and the golden-file loader."""
from __future__ import annotations

import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle

    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own host code, when oracle/_ref/libref.so was built (else the test skips)."""
    from oracle.oracle import Reference

    try:
        return Reference()
    except (FileNotFoundError, OSError) as exc:  # not built here, or its cudart is missing
        pytest.skip(f"reference oracle not available: {exc}")


def load_golden(name: str):
    path = os.path.join(GOLDEN, name)
    if name.endswith(".json"):
        with open(path) as f:
            return json.load(f)
    return dict(np.load(path))


@pytest.fixture(scope="session")
def golden():
    return load_golden

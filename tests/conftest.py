"""Test configuration: the ``gpu`` marker, import paths, shared fixtures.

Tests marked ``gpu`` call the CUDA kernels through the C ABI and need a B200;
everything else (oracle vs the reference's golden vectors, host logic, library
symbols) runs on CPU.
"""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir() -> Path:
    return REPO / "tests" / "golden"


@pytest.fixture(scope="session")
def reference_modules():
    """The reference's compiled CPU drivers (oracle/_ref), or skip when they were never built."""
    from oracle import build_ref

    try:
        build_ref.build()
        return {name: build_ref.load(name) for name in build_ref.MODULES}
    except FileNotFoundError as exc:  # neither the checkout nor a prebuilt module
        pytest.skip(str(exc))

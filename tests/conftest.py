"""pytest configuration: the `gpu` marker, and session fixtures for the package, the built CUDA
library and the CPU oracle."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def built_lib(pkg):
    """The in-tree shared library; built on demand (nvcc cross-compiles without a GPU)."""
    from ppl_nn_b200 import capi
    if not capi.LIB_PATH.exists():
        entry.build()
    return capi.library()


@pytest.fixture(scope="session")
def oracle_mod():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def orc(oracle_mod):
    oracle_mod.build()
    return oracle_mod.COracle()

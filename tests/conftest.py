"""pytest configuration: the ``gpu`` marker, the package alias and shared fixtures.

``-m "not gpu"`` tests run anywhere (they check the oracle, the host-side logic and that the C-ABI
library loads and exports what include/b200wmma.h declares).  ``-m gpu`` tests are the parity
tests: they call the CUDA kernels through the C ABI and compare with the CPU oracle.
"""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402

entry.load_package()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def oracle():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def lib(pkg):
    # built by __graft_entry__.build(); loading fails loudly if it is missing
    if not pkg._lib.LIB_PATH.exists():
        pkg.build.build()
    return pkg._lib.lib()


@pytest.fixture()
def handle(pkg, lib):
    """A fresh library handle on device 0 with a short wait budget, so that a pipeline bug
    surfaces as a reported timeout within a fraction of a second."""
    from cudanative_jl_b200.gemm import Handle

    h = Handle(0)
    h.set_option(pkg._lib.OPT_WAIT_BUDGET_NS, 200_000_000)
    yield h
    h.close()

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _ensure_built():
    lib = entry.PKG_DIR / "lib" / "libb200arrays.so"
    if not lib.exists():
        entry.build()


@pytest.fixture(scope="session")
def pkg():
    _ensure_built()
    return entry.load_package()


@pytest.fixture(scope="session")
def orc():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def gpu(pkg):
    """The package with device 0 selected; fails loudly when no device is present."""
    assert pkg.functional(), "GPU tests need a CUDA device and the built extension"
    pkg.device_(0)
    return pkg

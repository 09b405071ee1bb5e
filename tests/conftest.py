"""pytest configuration: the `gpu` marker and the package fixture."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as entry

    p = entry.load_package()
    p.load_library()
    return p


@pytest.fixture(scope="session")
def L(pkg):
    """The torch-facing operator mirror (sglang_cpp_b200.layers)."""
    return pkg.layers

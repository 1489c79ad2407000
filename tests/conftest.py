import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def port():
    from oracle import oracle as orc
    return orc.Port()


@pytest.fixture(scope="session")
def ref():
    """The reference's CPU backend compiled from its own sources; skipped where that build is absent."""
    from oracle import oracle as orc
    try:
        return orc.Ref()
    except FileNotFoundError as exc:
        pytest.skip(str(exc))


@pytest.fixture(scope="session")
def golden_dir():
    return ROOT / "tests" / "golden"

import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def library():
    """The built C-ABI library; built on first use where nvcc is available."""
    from turbogpt_b200 import bridge
    if not bridge.library_path().exists():
        from turbogpt_b200.build import build_library
        build_library()
    return bridge.load_library()


@pytest.fixture(scope="session")
def golden():
    return ROOT / "tests" / "golden"

import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def _ensure_built():
    from minicompiler_b200 import build

    if not build.LIB.exists():
        build.build_all()


@pytest.fixture(scope="session", autouse=True)
def built_library():
    _ensure_built()


@pytest.fixture(scope="session")
def mc():
    import minicompiler_b200

    return minicompiler_b200


@pytest.fixture(scope="session")
def oracle():
    from oracle import reference_cpu

    return reference_cpu


GOLDEN = Path(__file__).resolve().parent / "golden"

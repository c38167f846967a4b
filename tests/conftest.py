import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT / "kiln-compiler_b200", ROOT):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def plan_cases():
    return sorted(p.stem for p in (GOLDEN / "plans").glob("*.json"))


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN

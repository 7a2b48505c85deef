import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu); everything else runs on CPU")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure), built on demand."""
    from oracle import oracle as orc
    orc.lib()
    return orc


@pytest.fixture(scope="session")
def lb():
    import lithos_b200
    if not (ROOT / "lithos_b200" / "liblithos_b200.so").exists():
        lithos_b200.build()
    lithos_b200.lib()
    return lithos_b200


@pytest.fixture(scope="session")
def ctx(lb):
    """One device context for the whole GPU session (fails loudly without a GPU)."""
    c = lb.Context(0)
    yield c
    c.close()

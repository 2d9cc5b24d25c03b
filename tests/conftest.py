import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (runs the CUDA engine through the C ABI)")


@pytest.fixture(scope="session")
def lib():
    """The built engine library.  Never skipped: a missing library is a failure."""
    from metalium_rs_b200 import build, engine
    build.build()
    return engine.load_library()


@pytest.fixture(scope="session")
def eng(lib):
    """One engine on cuda:0 for the whole session (GPU tests only)."""
    from metalium_rs_b200 import CudaEngine
    e = CudaEngine(0)
    yield e
    e.close()


@pytest.fixture()
def fresh_eng(lib):
    """An engine of its own, for tests that leave a sticky device error behind."""
    from metalium_rs_b200 import CudaEngine
    e = CudaEngine(0)
    yield e
    e.close()

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def lib_built():
    """Builds libminit_b200.so if nvcc is present and it is stale; the package import fails loudly otherwise."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("minit_b200_build", os.path.join(ROOT, "minit_b200", "csrc", "build.py"))
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    build.build()
    return build.LIB

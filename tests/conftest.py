import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def built_lib():
    """Builds (if stale) and loads the CUDA library; a missing library is a hard failure."""
    from opfoundry_b200 import build
    build.build()
    from opfoundry_b200 import api
    return api.lib()


@pytest.fixture(scope="session")
def oracle():
    from oracle import build as obuild
    obuild.build_oracle()
    from oracle import oracle as O
    return O

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def sdk():
    from __graft_entry__ import load_package
    package = load_package()
    package.build_native()       # no-op when the in-tree artefact is current
    package.load_native()
    return package


@pytest.fixture(scope="session")
def oracle():
    from __graft_entry__ import load_oracle
    return load_oracle()[0]


@pytest.fixture(scope="session")
def oracle_c():
    from __graft_entry__ import load_oracle
    module = load_oracle()[1]
    module.build()
    return module


@pytest.fixture(scope="session")
def backend(sdk):
    import slidesparse_diffusion_b200.backend as module
    return module

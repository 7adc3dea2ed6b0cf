import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from __graft_entry__ import load_package  # noqa: E402

load_package()  # registers the package as module "mlel_b200" so that tests can import its submodules

# checkout of the reference project: present only where the fixtures were authored, never needed on a GPU box
REFERENCE_ROOT = os.environ.get("MLEL_REFERENCE_ROOT", "/root/reference")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def mlel():
    """The package, with its CUDA library loaded (fails loudly when the library is not built)."""
    pkg = load_package()
    pkg.lib()
    return pkg


@pytest.fixture(scope="session")
def reference_root():
    if not os.path.isdir(REFERENCE_ROOT):
        pytest.skip("reference checkout not present")
    return REFERENCE_ROOT


@pytest.fixture(autouse=True)
def _no_device_side_timeouts(request):
    """After every GPU test: no kernel may have given up on a bounded wait."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        assert load_package().lib().mlel_device_error() == 0, "a kernel recorded a timed-out wait"

import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def fixtures_json():
    with open(os.path.join(ROOT, "tests", "golden", "reference_fixtures.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def e2e_golden():
    with open(os.path.join(ROOT, "tests", "golden", "e2e_golden.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def port():
    from oracle import harness
    return harness.port()


@pytest.fixture(scope="session")
def ref_shim():
    from oracle import harness
    lib = harness.ref_shim()
    if lib is None:
        pytest.skip("oracle/_ref not built (reference sources absent)")
    return lib


@pytest.fixture(scope="session")
def ref_lib():
    from oracle import harness
    lib = harness.ref()
    if lib is None:
        pytest.skip("oracle/_ref not built (reference sources absent)")
    return lib


@pytest.fixture(scope="session")
def gpu_lib():
    """The product library. GPU tests fail loudly if it is missing or unbuilt."""
    from superslm_b200 import abi, build
    path = build.LIB
    if not os.path.exists(path):
        build.build()
    return abi.SslmLib(path)

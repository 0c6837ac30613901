import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def kat():
    import json
    with open(os.path.join(ROOT, "tests", "golden", "kat_nodes.json")) as f:
        return json.load(f)


@pytest.fixture()
def gpu():
    """The binding with a clean device status; asserts no kernel reported a timeout."""
    import torch
    import ginn_b200 as gb
    assert torch.cuda.is_available()
    # GINN_B200_TEST_PATH reruns the whole suite with another kernel choice as the default
    # (tests that pick a path themselves still override it).
    gb.set_option("force_path", int(os.environ.get("GINN_B200_TEST_PATH", "0")))
    gb.device_status(0, True)
    yield gb
    torch.cuda.synchronize()
    gb.set_option("force_path", 0)
    assert gb.device_status(0, True) == 0

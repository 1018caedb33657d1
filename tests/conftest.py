import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the built CUDA library")


@pytest.fixture(scope="session")
def oracle():
    from oracle.bindings import Oracle
    return Oracle()


def _ref(platform):
    from oracle.bindings import Ref
    try:
        return Ref(platform)
    except FileNotFoundError as e:  # the reference tree was never compiled on this machine
        pytest.skip(str(e))


@pytest.fixture(scope="session")
def ref():
    return _ref("ref")


@pytest.fixture(scope="session")
def zen2():
    return _ref("zen2")

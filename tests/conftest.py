import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

entry.load_package()  # registers the package as `hashattention_b200`


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture
def lib_option(pkg):
    """Sets dispatch options of the library (ha_set_option) for one test and puts the old values back."""
    from hashattention_b200 import _lib
    keys = {"cluster_gather": _lib.HA_OPT_CLUSTER_GATHER, "cluster_select": _lib.HA_OPT_CLUSTER_SELECT,
            "plan_handover": _lib.HA_OPT_PLAN_HANDOVER}
    lib = _lib.load()
    saved = {}

    def set_option(name, value):
        key = keys[name]
        saved.setdefault(key, lib.ha_get_option(key))
        assert lib.ha_set_option(key, int(value)) == _lib.HA_OK

    yield set_option
    for key, value in saved.items():
        lib.ha_set_option(key, value)

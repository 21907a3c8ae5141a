import importlib
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PKG_NAME = "mlsys-contest-syfi-agent-assisted_b200"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def pkg():
    return importlib.import_module(PKG_NAME)


@pytest.fixture(scope="session")
def oracle():
    return importlib.import_module("oracle.moe_oracle")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


_INPUT_CACHE = {}


@pytest.fixture(scope="session")
def make_inputs_cached(pkg):
    """Session cache of generated workloads keyed by their arguments (weights are costly to draw)."""

    def get(**kw):
        key = tuple(sorted(kw.items()))
        if key not in _INPUT_CACHE:
            if len(_INPUT_CACHE) >= 2:  # bound host/device memory held by the cache
                _INPUT_CACHE.pop(next(iter(_INPUT_CACHE)))
            _INPUT_CACHE[key] = pkg.make_inputs(**kw)
        return _INPUT_CACHE[key]

    return get

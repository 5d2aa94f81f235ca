import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_addoption(parser):
    parser.addoption("--zlm-bounds-check", action="store_true", default=False,
                     help="run against the bounds-check build of the kernel library: every call registers the "
                          "tensors it passes, and an access outside them fails the call")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200, sm_100a)")
    if config.getoption("--zlm-bounds-check"):
        from zlm_b200.kernels import set_build_variant
        set_build_variant("check")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA GPU here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)

"""Test configuration: the repository root on the path, the ``gpu`` marker, and
temporary model folders that are never committed."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_sessionfinish(session, exitstatus):
    """With IE_TEST_STATS=<file> set, what every comparison with the plain implementation measured is written there."""
    path = os.environ.get("IE_TEST_STATS")
    if not path:
        return
    import json

    import helpers
    with open(path, "w") as f:
        json.dump(helpers.STATS, f, indent=0)

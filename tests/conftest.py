"""Shared fixtures.  Tests marked ``gpu`` need a CUDA device (a B200); everything else runs on the
CPU.  Model folders are written to temporary folders and never kept."""
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


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """(name, dtype) -> folder of a tiny random model, made on first use."""
    import helpers
    made = {}

    def get(name: str, dtype: str) -> str:
        key = (name, dtype)
        if key not in made:
            d = tmp_path_factory.mktemp(f"{name}_{dtype}")
            made[key] = helpers.write_tiny(name, dtype, str(d))
        return made[key]
    return get

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, made once per session in a temporary folder."""
    import torch
    import helpers
    made = {}

    def get(name: str, dtype=torch.bfloat16, seed: int = 1, sharp: float = 1.0):
        key = (name, dtype, seed, sharp)
        if key not in made:
            d = str(tmp_path_factory.mktemp(f"{name}-{str(dtype).split('.')[-1]}-{seed}"))
            helpers.make_model_dir(helpers.TINY[name], d, seed=seed, dtype=dtype, sharp=sharp)
            made[key] = d
        return made[key]
    return get

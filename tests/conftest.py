import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs an sm_100a GPU (run with -m gpu)")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Writes tiny random model folders on demand: model_folders(name, dtype, std) -> path."""
    import helpers
    made = {}

    def get(name, dtype="float32", std=0.25, seed=None):
        key = (name, dtype, std, seed)
        if key not in made:
            d = tmp_path_factory.mktemp(f"{name}_{dtype}")
            helpers.write_tiny_model(str(d), name, dtype, std, seed)
            made[key] = str(d)
        return made[key]

    return get

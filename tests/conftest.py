import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, random weights, made once per test run."""
    import helpers
    out = {}
    for name in helpers.TINY:
        out[name] = helpers.make_model_dir(str(tmp_path_factory.mktemp(f"model_{name}")), name)
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    """name -> (config dict, float64 tensors) as the plain implementation reads them."""
    import plain_llama
    return {name: plain_llama.read_model(path) for name, path in model_dirs.items()}

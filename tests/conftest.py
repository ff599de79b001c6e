import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    # the file that must be collected last stays last whatever the order of discovery
    items.sort(key=lambda item: item.fspath.basename.startswith("test_zz"))


@pytest.fixture(scope="session")
def tiny_models(tmp_path_factory):
    """Model folders of the tiny configurations, made once per session in a temporary folder."""
    import helpers
    root = tmp_path_factory.mktemp("models")
    return {name: helpers.make_model(str(root / name), name) for name in helpers.TINY}


@pytest.fixture(autouse=True)
def _no_model_carried_over():
    """The 32-bit tolerance follows the model that the test last asked the plain implementation about."""
    import helpers
    helpers._LAST_MODEL["longest_sum"] = None
    yield

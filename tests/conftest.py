"""Shared pytest setup: marker registration and import paths.

`gpu` tests need a B200 and call the CUDA library through its C-ABI; everything
else runs on CPU.  The oracle under oracle/ is imported here only as the checker.
"""
import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def load_package():
    """Imports the hyphen-named package directory under the module name `itex_b200`."""
    if "itex_b200" in sys.modules:
        return sys.modules["itex_b200"]
    pkg_dir = os.path.join(ROOT, "intel-extension-for-tensorflow_b200")
    spec = importlib.util.spec_from_file_location(
        "itex_b200", os.path.join(pkg_dir, "__init__.py"), submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["itex_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def itex():
    return load_package()


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN

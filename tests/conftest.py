"""pytest configuration: the `gpu` marker, import paths, and shared helpers.

Layout of what the tests use:
  - `w4a8`   : the package's ctypes binding of libw4a8_b200.so (dgx-serving_b200/__init__.py)
  - `oracle` : the CPU restatement of the reference path (oracle/oracle.py; test infrastructure)
"""
import importlib.util
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, ROOT)


def load_package():
    """The package directory is named dgx-serving_b200 (not an identifier); import it as dgx_serving_b200."""
    name = "dgx_serving_b200"
    if name in sys.modules:
        return sys.modules[name]
    path = os.path.join(ROOT, "dgx-serving_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=[os.path.dirname(path)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def w4a8():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    return torch.device("cuda:0")


def to_dev(a, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

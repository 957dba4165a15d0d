import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def load_package():
    """The package directory is named cl-eden-kernel_b200 (not an identifier), so import it by path."""
    name = "cl_eden_kernel_b200"
    if name in sys.modules:
        return sys.modules[name]
    path = os.path.join(ROOT, "cl-eden-kernel_b200", "__init__.py")
    if not os.path.exists(os.path.join(ROOT, "cl-eden-kernel_b200", "libenn_b200.so")):
        import subprocess
        subprocess.run(["make", "-C", os.path.join(ROOT, "cl-eden-kernel_b200"), "-j8"], check=True, capture_output=True)
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=[os.path.dirname(path)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def enn():
    return load_package()


@pytest.fixture(scope="session")
def orc():
    from oracle import orc as o
    return o


@pytest.fixture(scope="session")
def ctx(enn):
    c = enn.Context(0)
    yield c
    c.close()

import importlib.util
import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PACKAGE = os.path.join(REPO, "transformer-in-c_b200")
# The reference's unmodified host code, compiled twice (oracle/build_ref.py):
# the copy that drives the backend, and the copy that only ever runs the CPU
# loops and serves as the checker.
HOST_LIBRARY = os.path.join(PACKAGE, "host", "libvithost.so")
CHECKER_LIBRARY = os.path.join(REPO, "oracle", "_ref", "libvithost.so")
GOLDEN = os.path.join(REPO, "tests", "golden")

if REPO not in sys.path:
    sys.path.insert(0, REPO)


def load_module(name, path):
    """The package directory is not a valid Python identifier, so its modules
    are loaded by path."""
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200")


@pytest.fixture(scope="session")
def vit_host_module():
    return load_module("vitb200_vit_host", os.path.join(PACKAGE, "vit_host.py"))


@pytest.fixture(scope="session")
def host_lib(vit_host_module):
    if not os.path.exists(HOST_LIBRARY):
        pytest.skip("host/libvithost.so not built (needs the reference tree)")
    return vit_host_module.load_host_library(HOST_LIBRARY)


@pytest.fixture(scope="session")
def checker_lib(vit_host_module):
    """The reference's CPU path in a library of its own: no backend is ever
    installed into it, whatever the state of the one the tests drive."""
    if not os.path.exists(CHECKER_LIBRARY):
        pytest.skip("oracle/_ref/libvithost.so not built (needs the reference tree)")
    return vit_host_module.load_host_library(CHECKER_LIBRARY,
                                             visible_to_backend=False)


@pytest.fixture(scope="session")
def backend(vit_host_module, host_lib):
    """One backend for the whole GPU session; raises (does not skip) when the
    library or the device is missing."""
    instance = vit_host_module.Backend()
    yield instance
    instance.disable()
    instance.close()

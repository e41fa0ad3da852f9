"""Shared fixtures.  `-m "not gpu"` runs on a CPU-only box; `-m gpu` needs a B200."""
import ctypes
import importlib.util
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "pulp-trainlib_b200")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselected on CPU-only boxes")


def load_pkg():
    """Import the package directory (its name has a hyphen) as module `pulp_trainlib_b200`."""
    if "pulp_trainlib_b200" in sys.modules:
        return sys.modules["pulp_trainlib_b200"]
    spec = importlib.util.spec_from_file_location(
        "pulp_trainlib_b200", os.path.join(PKG_DIR, "__init__.py"), submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["pulp_trainlib_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def pkg():
    return load_pkg()


@pytest.fixture(scope="session")
def oracle():
    """The CPU restatement (oracle/liboracle.so), built on demand with gcc."""
    import oracle_bind
    return oracle_bind.load()


@pytest.fixture(scope="session")
def reflib(pkg):
    """The reference's own C sources compiled for the host (oracle/_ref/libpulp_ref.so)."""
    path = os.path.join(ROOT, "oracle", "_ref", "libpulp_ref.so")
    if not os.path.exists(path):
        if os.path.isdir(os.path.join(os.environ.get("TRAINLIB_REF", os.path.join(ROOT, "..", "reference")), "lib", "sources")):
            subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "ref"], stdout=subprocess.DEVNULL)
        else:
            pytest.skip("oracle/_ref/libpulp_ref.so not built (needs the reference sources)")
    return pkg.bind(ctypes.CDLL(path))


@pytest.fixture(scope="session")
def gpulib(pkg):
    """libtrainlib_b200.so on a live device.  A missing library or device is a failure, not a skip."""
    lib = pkg.load()
    rc = lib.trainlib_init(-1)
    assert rc == 0, "trainlib_init failed: %s" % lib.trainlib_last_error_string().decode()
    return lib

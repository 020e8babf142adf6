import importlib
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = "heterogeneity-aware-lowering-and-optimization_b200"
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    return importlib.import_module(PKG)


@pytest.fixture(scope="session")
def odla(pkg):
    return pkg.odla


@pytest.fixture(scope="session")
def models():
    class M:
        mnist = importlib.import_module(PKG + ".halo_models.mnist")
        resnet50 = importlib.import_module(PKG + ".halo_models.resnet50")
        yolov3 = importlib.import_module(PKG + ".halo_models.yolov3")
        bert = importlib.import_module(PKG + ".halo_models.bert")
    return M


@pytest.fixture(scope="session")
def lib(pkg):
    """libodla_b200.so; built on demand (nvcc cross-compiles without a GPU)."""
    if not os.path.exists(pkg.default_library_path()):
        pkg.build.build()
    return pkg.load()


@pytest.fixture(scope="session")
def ref(odla):
    """The CPU oracle platform (oracle/libodla_cpuref.so); built on demand with gcc."""
    path = os.path.join(ROOT, "oracle", "libodla_cpuref.so")
    if not os.path.exists(path):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True)
    return odla.OdlaLib(path)


@pytest.fixture(scope="session")
def gpu_lib(lib):
    if lib.b200_DeviceCount() < 1:
        pytest.fail("a test marked gpu ran without a CUDA device")
    return lib

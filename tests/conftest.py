import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "onnx-mlir_b200"))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def built():
    """Builds (or reuses) the library and the oracle; returns their paths."""
    sys.path.insert(0, ROOT)
    import importlib.util
    def load(name, path):
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod
    lib = load("omcuda_build", os.path.join(ROOT, "onnx-mlir_b200", "build.py")).build_lib()
    ob = load("oracle_build", os.path.join(ROOT, "oracle", "build.py"))
    return {"lib": lib, "oracle": ob.build_oracle(), "ref_runtime": ob.build_ref_runtime()}


@pytest.fixture(scope="session")
def orc(built):
    import oracle_lib
    return oracle_lib.Oracle(built["oracle"])


@pytest.fixture(scope="session")
def omcuda(built):
    import omcuda as m
    m.lib()
    return m


@pytest.fixture(scope="session")
def gpu(omcuda):
    """The library initialised on a B200; GPU tests fail (not skip) without it."""
    omcuda.init()
    return omcuda

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
    spec = importlib.util.spec_from_file_location(
        "omcuda_build", os.path.join(ROOT, "onnx-mlir_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    lib, orc, ref = mod.build_all()
    return {"lib": lib, "oracle": orc, "ref_runtime": ref}


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

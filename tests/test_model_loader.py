"""Compiled-model artefacts and their loader without a GPU: the model builder
produces a .so with the entry points and signatures of an onnx-mlir model and
an external constants file; the session loader opens it by tag, answers the
queries, and a run without a B200 fails the way the reference reports failure
(NULL from run_main_graph, errno set) instead of computing anything on the
CPU."""
import ctypes
import os

import numpy as np
import pytest

from omcuda.synthetic import make_encoder


@pytest.fixture(scope="module")
def models(tmp_path_factory, omcuda):
    from omcuda import model_builder
    d = str(tmp_path_factory.mktemp("models"))
    rng = np.random.default_rng(5)
    W = rng.integers(-127, 128, (96, 40), dtype=np.int8)
    bias = rng.normal(0, 0.02, 40).astype(np.float32)
    lin = model_builder.build_dyn_quant_linear_model(d, "Linear", W, 0.0157, bias)
    enc = model_builder.build_encoder_model(d, "enc", 128, 2, 256, make_encoder(3, 128, 256, 2))
    return {"dir": d, "linear": lin, "encoder": enc, "W": W, "bias": bias}


def test_model_exports_the_reference_entry_points(models):
    so = ctypes.CDLL(models["linear"])
    for sym in ("run_main_graph", "run_main_graph_linear", "omQueryEntryPoints",
                "omQueryEntryPoints_linear", "omInputSignature", "omInputSignature_linear",
                "omOutputSignature", "omOutputSignature_linear"):
        assert hasattr(so, sym), sym
    assert os.path.exists(os.path.join(models["dir"], "Linear.constants.bin"))
    # the weights are in the constants file, not in the library
    blob = open(os.path.join(models["dir"], "Linear.constants.bin"), "rb").read()
    assert blob[:models["W"].size] == models["W"].tobytes()
    assert os.path.getsize(models["linear"]) < 200_000


def test_session_queries(models, omcuda):
    from omcuda.session import OMExecutionSession, parse_signature
    s = OMExecutionSession(models["linear"])          # tag from the file name
    assert s.entry_points() == ["run_main_graph_linear"]
    (dt, dims, name), = parse_signature(s.input_signature())
    assert dt == np.float32 and dims == [-1, 96] and name == "X"
    (dt, dims, name), = parse_signature(s.output_signature())
    assert dims == [-1, 40] and name == "Y"
    s.set_entry_point("run_main_graph")
    with pytest.raises(omcuda.OmcudaError):
        s.set_entry_point("no_such_entry")
    s.close()
    s = OMExecutionSession(models["linear"], tag="NONE")   # unsuffixed symbols
    assert "768" not in s.input_signature()
    s.close()
    with pytest.raises(omcuda.OmcudaError):
        OMExecutionSession(models["linear"], tag="wrongtag")
    with pytest.raises(omcuda.OmcudaError):
        OMExecutionSession(os.path.join(models["dir"], "missing.so"))


def test_constants_path_rule(models, omcuda, tmp_path, monkeypatch):
    # The constants file is found through OM_CONSTANT_PATH, which the loader
    # points at the model's folder unless the caller set it.
    L = omcuda.lib()
    L.omcudaLoadConstantData.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p,
                                         ctypes.c_int64, ctypes.c_int64]
    L.omcudaUnloadConstantData.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64]
    monkeypatch.setenv("OM_CONSTANT_PATH", models["dir"])
    addr = ctypes.c_void_p()
    size = os.path.getsize(os.path.join(models["dir"], "Linear.constants.bin"))
    assert L.omcudaLoadConstantData(ctypes.byref(addr), b"Linear.constants.bin", size, 1) == 0
    assert ctypes.string_at(addr.value, 16) == models["W"].tobytes()[:16]
    assert L.omcudaUnloadConstantData(ctypes.byref(addr), size) == 0 and not addr.value
    monkeypatch.setenv("OM_CONSTANT_PATH", str(tmp_path))
    assert L.omcudaLoadConstantData(ctypes.byref(addr), b"Linear.constants.bin", size, 1) != 0
    L.omcudaClearError()
    # big-endian packs are refused on this little-endian host
    monkeypatch.setenv("OM_CONSTANT_PATH", models["dir"])
    assert L.omcudaLoadConstantData(ctypes.byref(addr), b"Linear.constants.bin", size, 0) != 0
    L.omcudaClearError()


def test_run_without_gpu_fails_like_the_reference(models, omcuda):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: covered by the GPU tests")
    from omcuda.session import OMExecutionSession
    s = OMExecutionSession(models["encoder"])
    with pytest.raises(omcuda.OmcudaError):
        s.run([np.zeros((1, 8, 128), np.float32)])
    s.close()


def test_cuda_array_interface_objects_are_checked_before_wrapping():
    # The zero-copy wrapper of foreign device buffers refuses what it cannot
    # describe as a dense OMTensor (no GPU needed to say no).
    import numpy as np
    import pytest
    import omcuda

    class Fake:
        def __init__(self, **cai):
            self.__cuda_array_interface__ = dict(version=2, data=(4096, False), **cai)

    with pytest.raises(ValueError):
        omcuda.Tensor.from_cuda_array(Fake(shape=(4, 4), typestr="<f4", strides=(4, 16)))
    with pytest.raises(TypeError):
        omcuda.Tensor.from_cuda_array(Fake(shape=(4,), typestr="<c8", strides=None))
    host = omcuda.Tensor.__new__(omcuda.Tensor)
    host.handle, host.array, host.device, host.borrowed = None, None, False, False
    assert not hasattr(host, "__cuda_array_interface__")

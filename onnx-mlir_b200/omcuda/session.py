"""OMExecutionSession: the Python loader of compiled models, with the interface
of onnx-mlir's PyRuntime (src/Runtime/python/PyExecutionSession.cpp:129-395:
OMExecutionSession(shared_lib_path, tag, use_default_entry_point), run,
entry_points, set_entry_point, input_signature, output_signature), on top of
the library's omcudaSession* C API.  Device-aware: run() takes numpy arrays
(host tensors, results come back as numpy arrays) or omcuda.Tensor objects
(passed as they are; device tensors in give device tensors out, so that models
can be chained without touching host memory) or any object with
__cuda_array_interface__, e.g. a torch.Tensor on the GPU (wrapped without a
copy; device results expose the same interface, so torch.as_tensor(result,
device="cuda") is a view, not a copy)."""
import ctypes
import json

import numpy as np

from . import _OM2NP, OmcudaError, Tensor, check, lib, ECUDA


def _bind():
    L = lib()
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    L.omcudaSessionCreate.restype = vp
    L.omcudaSessionCreate.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int]
    L.omcudaSessionQueryEntryPoints.restype = ctypes.POINTER(ctypes.c_char_p)
    L.omcudaSessionQueryEntryPoints.argtypes = [vp, ctypes.POINTER(i64)]
    L.omcudaSessionSetEntryPoint.argtypes = [vp, ctypes.c_char_p]
    L.omcudaSessionInputSignature.restype = ctypes.c_char_p
    L.omcudaSessionInputSignature.argtypes = [vp]
    L.omcudaSessionOutputSignature.restype = ctypes.c_char_p
    L.omcudaSessionOutputSignature.argtypes = [vp]
    L.omcudaSessionRun.restype = vp
    L.omcudaSessionRun.argtypes = [vp, vp]
    L.omcudaSessionDestroy.argtypes = [vp]
    return L


class OMExecutionSession:
    def __init__(self, shared_lib_path, tag="", use_default_entry_point=True):
        self.L = _bind()
        self.handle = self.L.omcudaSessionCreate(shared_lib_path.encode(), tag.encode(),
                                                 int(use_default_entry_point))
        if not self.handle:
            check()
            raise OmcudaError(ECUDA, "cannot load model " + shared_lib_path)

    def entry_points(self):
        n = ctypes.c_int64()
        arr = self.L.omcudaSessionQueryEntryPoints(self.handle, ctypes.byref(n))
        return [arr[i].decode() for i in range(n.value)]

    def set_entry_point(self, name):
        if self.L.omcudaSessionSetEntryPoint(self.handle, name.encode()) != 0:
            check()

    def input_signature(self):
        s = self.L.omcudaSessionInputSignature(self.handle)
        if s is None:
            check()
        return s.decode()

    def output_signature(self):
        s = self.L.omcudaSessionOutputSignature(self.handle)
        if s is None:
            check()
        return s.decode()

    def run(self, inputs):
        """inputs: list of numpy arrays and / or omcuda.Tensor objects.  Returns
        a list: numpy arrays for host results, Tensors for device results."""
        L = self.L
        ts = [x if isinstance(x, Tensor)
              else Tensor.from_cuda_array(x) if hasattr(x, "__cuda_array_interface__")
              else Tensor.from_numpy(np.asarray(x)) for x in inputs]
        arr = (ctypes.c_void_p * max(len(ts), 1))(*[t.handle for t in ts])
        ins = L.omTensorListCreate(arr, len(ts))
        ctypes.set_errno(0)
        outs = L.omcudaSessionRun(self.handle, ins)
        L.omTensorListDestroyShallow(ins)
        if not outs:
            check()
            raise OmcudaError(ECUDA, "run_main_graph returned NULL")
        res = []
        for i in range(L.omTensorListGetSize(outs)):
            o = L.omTensorListGetOmtByIndex(outs, i)
            if L.omcudaTensorIsOnDevice(o):
                res.append(Tensor(o, None, True))
                continue
            n = L.omTensorGetNumElems(o)
            rank = L.omTensorGetRank(o)
            shp = L.omTensorGetShape(o)
            shape = tuple(int(shp[k]) for k in range(rank))
            dt = _OM2NP[L.omTensorGetDataType(o)]
            buf = (ctypes.c_char * max(L.omTensorGetBufferSize(o), 1)).from_address(
                L.omTensorGetDataPtr(o))
            res.append(np.frombuffer(buf, dtype=dt, count=int(n)).reshape(shape).copy())
            L.omTensorDestroy(o)
        L.omTensorListDestroyShallow(outs)
        return res

    def close(self):
        if self.handle:
            self.L.omcudaSessionDestroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def parse_signature(sig):
    """[(numpy dtype, dims with -1 for dynamic, name)] of a signature string."""
    names = {"f32": np.float32, "ui8": np.uint8, "i8": np.int8, "i32": np.int32,
             "i64": np.int64, "ui16": np.uint16}
    return [(np.dtype(names[e["type"]]), [int(d) for d in e["dims"]], e.get("name", ""))
            for e in json.loads(sig)]

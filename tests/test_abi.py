"""The C ABI of libomcuda without a GPU: the library loads, exports every
symbol include/*.h declares, implements the OMTensor runtime compatibly with
the reference's own (when that was built from the reference tree), and fails
loudly instead of falling back when no GPU is present."""
import ctypes
import errno
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    syms = set()
    for name in os.listdir(os.path.join(ROOT, "include")):
        if not name.endswith(".h"):
            continue
        text = open(os.path.join(ROOT, "include", name)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"#.*", "", text)
        for m in re.finditer(r"\b((?:om|OM)\w+)\s*\(", text):
            syms.add(m.group(1))
        for m in re.finditer(r"extern\s+long\s+(\w+)\s*;", text):
            syms.add(m.group(1))
    return sorted(syms)


def test_every_declared_symbol_is_exported(built):
    L = ctypes.CDLL(built["lib"])
    syms = declared_symbols()
    assert len(syms) > 60
    missing = [s for s in syms if not hasattr(L, s)]
    assert not missing, missing


def test_omtensor_runtime_host_only(omcuda):
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    t = omcuda.Tensor.from_numpy(a)
    L = omcuda.lib()
    assert t.shape == (2, 3, 4)
    st = L.omTensorGetStrides(t.handle)
    assert [st[i] for i in range(3)] == [12, 4, 1]
    assert L.omTensorGetNumElems(t.handle) == 24
    assert L.omTensorGetBufferSize(t.handle) == 96
    assert L.omTensorGetDataPtr(t.handle) == a.ctypes.data
    arr = (ctypes.c_void_p * 2)(t.handle, t.handle)
    lst = L.omTensorListCreate(arr, 2)
    assert L.omTensorListGetSize(lst) == 2
    assert L.omTensorListGetOmtByIndex(lst, 1) == t.handle
    assert L.omTensorListGetOmtByIndex(lst, 2) is None
    L.omTensorListDestroyShallow(lst)
    e = omcuda.Tensor(L.omTensorCreateEmpty((ctypes.c_int64 * 1)(5), 1, omcuda.ONNX_INT32))
    assert L.omTensorGetBufferSize(e.handle) == 20


def test_struct_layout_matches_reference_runtime(built, omcuda):
    """Tensors made by onnx-mlir's own libcruntime are read by ours and vice
    versa: the krnl.call wrappers a compiled model passes come from theirs."""
    if not built["ref_runtime"] or not os.path.exists(built["ref_runtime"]):
        pytest.skip("reference runtime not built (no onnx-mlir tree on this machine)")
    R = ctypes.CDLL(built["ref_runtime"])
    L = omcuda.lib()
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    for lib in (R,):
        lib.omTensorCreate.restype = vp
        lib.omTensorCreate.argtypes = [vp, ctypes.POINTER(i64), i64, ctypes.c_int]
        lib.omTensorGetDataPtr.restype = vp
        lib.omTensorGetDataPtr.argtypes = [vp]
        lib.omTensorGetShape.restype = ctypes.POINTER(i64)
        lib.omTensorGetShape.argtypes = [vp]
        lib.omTensorGetStrides.restype = ctypes.POINTER(i64)
        lib.omTensorGetStrides.argtypes = [vp]
        lib.omTensorGetRank.restype = i64
        lib.omTensorGetRank.argtypes = [vp]
        lib.omTensorGetDataType.argtypes = [vp]
        lib.omTensorGetNumElems.restype = i64
        lib.omTensorGetNumElems.argtypes = [vp]
        lib.omTensorGetBufferSize.restype = i64
        lib.omTensorGetBufferSize.argtypes = [vp]
        lib.omTensorGetOwning.restype = i64
        lib.omTensorGetOwning.argtypes = [vp]
        lib.omTensorDestroy.argtypes = [vp]
        lib.omTensorListCreate.restype = vp
        lib.omTensorListCreate.argtypes = [ctypes.POINTER(vp), i64]
        lib.omTensorListGetSize.restype = i64
        lib.omTensorListGetSize.argtypes = [vp]
        lib.omTensorListGetOmtByIndex.restype = vp
        lib.omTensorListGetOmtByIndex.argtypes = [vp, i64]
        lib.omTensorListDestroyShallow.argtypes = [vp]
    L.omTensorGetOwning.restype = i64
    L.omTensorGetOwning.argtypes = [vp]
    a = np.arange(30, dtype=np.uint8).reshape(5, 6)
    shape = (i64 * 2)(5, 6)
    # theirs -> ours
    t = R.omTensorCreate(a.ctypes.data, shape, 2, omcuda.ONNX_UINT8)
    assert L.omTensorGetRank(t) == 2
    assert [L.omTensorGetShape(t)[i] for i in range(2)] == [5, 6]
    assert [L.omTensorGetStrides(t)[i] for i in range(2)] == [6, 1]
    assert L.omTensorGetDataType(t) == omcuda.ONNX_UINT8
    assert L.omTensorGetDataPtr(t) == a.ctypes.data
    assert L.omTensorGetBufferSize(t) == 30 and L.omTensorGetOwning(t) == 0
    lst = R.omTensorListCreate((vp * 1)(t), 1)
    assert L.omTensorListGetSize(lst) == 1 and L.omTensorListGetOmtByIndex(lst, 0) == t
    L.omTensorListDestroyShallow(lst)
    L.omTensorDestroy(t)
    # ours -> theirs
    t = L.omTensorCreate(a.ctypes.data, shape, 2, omcuda.ONNX_UINT8)
    assert R.omTensorGetRank(t) == 2
    assert [R.omTensorGetShape(t)[i] for i in range(2)] == [5, 6]
    assert [R.omTensorGetStrides(t)[i] for i in range(2)] == [6, 1]
    assert R.omTensorGetDataType(t) == omcuda.ONNX_UINT8
    assert R.omTensorGetDataPtr(t) == a.ctypes.data
    assert R.omTensorGetNumElems(t) == 30 and R.omTensorGetOwning(t) == 0
    lst = L.omTensorListCreate((vp * 1)(t), 1)
    assert R.omTensorListGetSize(lst) == 1 and R.omTensorListGetOmtByIndex(lst, 0) == t
    R.omTensorListDestroyShallow(lst)
    R.omTensorDestroy(t)


def _no_gpu():
    try:
        import torch
        return not torch.cuda.is_available()
    except Exception:
        return True


@pytest.mark.skipif(not _no_gpu(), reason="checks the behaviour on a machine without a GPU")
def test_no_gpu_means_loud_failure_not_fallback(omcuda):
    L = omcuda.lib()
    L.omcudaClearError()
    x = np.ones((4, 4), np.float32)
    with pytest.raises(omcuda.OmcudaError) as ei:
        omcuda.dynamic_quantize_linear(x)
    assert ei.value.code == omcuda.ECUDA
    # the accelerator gate the generated entry point calls reports EPERM
    ctypes.set_errno(0)
    assert L.OMInitCompatibleAccelCUDA(0x000100) == 0
    L.omcudaClearError()
    # a model compiled for a newer library is refused even before touching a GPU
    assert L.OMInitCompatibleAccelCUDA(0x010000) == 0
    L.omcudaClearError()


def test_sticky_error_blocks_later_calls(omcuda):
    L = omcuda.lib()
    L.omcudaClearError()
    x = omcuda.Tensor.from_numpy(np.ones(4, np.float32))
    y = omcuda.Tensor.from_numpy(np.ones(4, np.uint8))
    s = omcuda.Tensor.from_numpy(np.zeros((), np.float32))
    z = omcuda.Tensor.from_numpy(np.zeros((), np.uint8))
    L.omcudaDynamicQuantizeLinear(y.handle, s.handle, z.handle, None)
    first = L.omcudaGetLastError()
    assert first != omcuda.OK
    msg = L.omcudaGetLastErrorString()
    L.omcudaDynamicQuantizeLinear(y.handle, s.handle, z.handle, x.handle)
    assert L.omcudaGetLastError() == first and L.omcudaGetLastErrorString() == msg
    L.omcudaClearError()
    assert L.omcudaGetLastError() == omcuda.OK

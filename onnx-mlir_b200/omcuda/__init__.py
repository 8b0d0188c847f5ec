"""ctypes host binding of libomcuda.

This is the Python mirror of the reference's loaders (the role
src/Runtime/python/PyExecutionSession.cpp plays for a compiled model): it
builds OMTensor wrappers over numpy arrays, calls the library's krnl.call-level
entry points, and turns the library's sticky status into exceptions.  All
arithmetic happens in the CUDA library; there is no Python or CPU fallback, and
importing succeeds without a GPU only so that the ABI can be inspected -- every
compute call raises OmcudaError when no B200 is present.
"""
import ctypes
import os

import numpy as np

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "lib", "libomcuda.so")

# ONNX TensorProto.DataType values used by OMTensor
# (include/onnx-mlir/Runtime/OnnxDataTypeMetaData.inc:24-45 in onnx-mlir).
ONNX_FLOAT, ONNX_UINT8, ONNX_INT8, ONNX_UINT16, ONNX_INT32, ONNX_INT64 = 1, 2, 3, 4, 6, 7
_NP2OM = {
    np.dtype(np.float32): ONNX_FLOAT,
    np.dtype(np.uint8): ONNX_UINT8,
    np.dtype(np.int8): ONNX_INT8,
    np.dtype(np.uint16): ONNX_UINT16,
    np.dtype(np.int32): ONNX_INT32,
    np.dtype(np.int64): ONNX_INT64,
}
_OM2NP = {v: k for k, v in _NP2OM.items()}

OK, EINVAL, ENOMEM, ECUDA, ETIMEDOUT, ENOTSUP = range(6)


def _c(a, dtype=None):
    """C-contiguous view/copy that keeps rank-0 arrays rank 0."""
    return np.require(a, dtype=dtype, requirements="C")


class OmcudaError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("omcuda error %d: %s" % (code, msg))
        self.code = code


_lib = None


def lib():
    """Loads libomcuda.so; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(
                "%s is missing: run `python onnx-mlir_b200/build.py`" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        L.omTensorCreate.restype = vp
        L.omTensorCreate.argtypes = [vp, ctypes.POINTER(i64), i64, i32]
        L.omTensorCreateEmpty.restype = vp
        L.omTensorCreateEmpty.argtypes = [ctypes.POINTER(i64), i64, i32]
        L.omTensorDestroy.argtypes = [vp]
        L.omTensorGetDataPtr.restype = vp
        L.omTensorGetDataPtr.argtypes = [vp]
        L.omTensorGetShape.restype = ctypes.POINTER(i64)
        L.omTensorGetShape.argtypes = [vp]
        L.omTensorGetStrides.restype = ctypes.POINTER(i64)
        L.omTensorGetStrides.argtypes = [vp]
        L.omTensorGetRank.restype = i64
        L.omTensorGetRank.argtypes = [vp]
        L.omTensorGetDataType.restype = i32
        L.omTensorGetDataType.argtypes = [vp]
        L.omTensorGetNumElems.restype = i64
        L.omTensorGetNumElems.argtypes = [vp]
        L.omTensorGetBufferSize.restype = i64
        L.omTensorGetBufferSize.argtypes = [vp]
        L.omTensorListCreate.restype = vp
        L.omTensorListCreate.argtypes = [ctypes.POINTER(vp), i64]
        L.omTensorListDestroy.argtypes = [vp]
        L.omTensorListDestroyShallow.argtypes = [vp]
        L.omTensorListGetSize.restype = i64
        L.omTensorListGetSize.argtypes = [vp]
        L.omTensorListGetOmtByIndex.restype = vp
        L.omTensorListGetOmtByIndex.argtypes = [vp, i64]
        L.omcudaGetLastError.restype = i32
        L.omcudaGetLastErrorString.restype = ctypes.c_char_p
        L.OMInitCompatibleAccelCUDA.restype = ctypes.c_uint64
        L.OMInitCompatibleAccelCUDA.argtypes = [ctypes.c_uint64]
        L.omcudaTensorCreateOnDevice.restype = vp
        L.omcudaTensorCreateOnDevice.argtypes = [ctypes.POINTER(i64), i64, i32]
        L.omcudaTensorToDevice.restype = vp
        L.omcudaTensorToDevice.argtypes = [vp]
        L.omcudaTensorToHost.restype = vp
        L.omcudaTensorToHost.argtypes = [vp]
        L.omcudaTensorDestroy.argtypes = [vp]
        L.omcudaTensorIsOnDevice.restype = i32
        L.omcudaTensorIsOnDevice.argtypes = [vp]
        L.omcudaHostAlloc.restype = vp
        L.omcudaHostAlloc.argtypes = [i64]
        L.omcudaHostFree.argtypes = [vp]
        L.omcudaDeviceAlloc.restype = vp
        L.omcudaDeviceAlloc.argtypes = [i64]
        L.omcudaDeviceFree.argtypes = [vp]
        L.omcudaGetStream.restype = vp
        L.omcudaStreamCreate.restype = vp
        L.omcudaStreamDestroy.argtypes = [vp]
        L.omcudaSetStream.argtypes = [vp]
        L.omcudaRegisterConstant.argtypes = [vp]
        L.omcudaLaunchCount.restype = i64
        L.omcudaSetQuantizationMode.argtypes = [i64]
        L.omcudaSetQuantizationMode.restype = None
        L.omcudaGetQuantizationMode.restype = i64
        for name, n in (("omcudaDynamicQuantizeLinear", 4),
                        ("omcudaQuantizeLinear", 4),
                        ("omcudaMatMulInteger", 5), ("omcudaQLinearMatMul", 9),
                        ("omcudaDequantizeLinear", 4), ("omcudaGelu", 2),
                        ("omcudaAdd", 3), ("omcudaTranspose0213", 2),
                        ("omcudaMatMulF32", 3)):
            getattr(L, name).argtypes = [vp] * n
            getattr(L, name).restype = None
        L.omcudaDynQuantLinear.argtypes = [vp] * 6 + [i64]
        L.omcudaDynQuantLinear.restype = None
        L.omcudaSoftmax.argtypes = [vp, vp, i64]
        L.omcudaSoftmax.restype = None
        L.omcudaLayerNormalization.argtypes = [vp, vp, vp, vp, i64,
                                               ctypes.c_double]
        L.omcudaLayerNormalization.restype = None
        L.omcudaAttention.argtypes = [vp, vp, vp, vp, i64, ctypes.c_double]
        L.omcudaAttention.restype = None
        _lib = L
    return _lib


def check():
    """Raises (and clears) the calling thread's sticky library status."""
    L = lib()
    code = L.omcudaGetLastError()
    if code != OK:
        msg = L.omcudaGetLastErrorString().decode()
        L.omcudaClearError()
        raise OmcudaError(code, msg)


def init(version=0x000100):
    """OMInitCompatibleAccelCUDA, as the generated run_main_graph calls it."""
    ok = lib().OMInitCompatibleAccelCUDA(version)
    if not ok:
        check()
        raise OmcudaError(ECUDA, "OMInitCompatibleAccelCUDA refused (EPERM)")


def synchronize():
    lib().omcudaSynchronize()
    check()


def launch_count():
    return int(lib().omcudaLaunchCount())


class Tensor:
    """An OMTensor wrapper.  Host tensors keep their numpy array alive; device
    tensors own a buffer from the library pool."""

    def __init__(self, handle, array=None, device=False, borrowed=False):
        self.handle = handle
        self.array = array
        self.device = device
        self.borrowed = borrowed  # a device buffer owned by someone else

    @staticmethod
    def from_cuda_array(obj):
        """Zero-copy view of a device buffer some other library owns: any object
        with __cuda_array_interface__ (a torch.Tensor on the GPU, a cupy array).
        The OMTensor is non-owning and keeps `obj` alive; the caller orders the
        two libraries' streams (run on the same stream via set_stream, or
        synchronize in between)."""
        cai = obj.__cuda_array_interface__
        if cai.get("strides") is not None:
            raise ValueError("from_cuda_array needs a contiguous (C-order) buffer")
        dt = np.dtype(cai["typestr"])
        if dt not in _NP2OM:
            raise TypeError("unsupported element type %s" % dt)
        shape_t = tuple(int(d) for d in cai["shape"])
        shape = (ctypes.c_int64 * max(len(shape_t), 1))(*shape_t)
        ptr = ctypes.c_void_p(int(cai["data"][0]))
        h = lib().omTensorCreate(ptr, shape, len(shape_t), _NP2OM[dt])
        if not h:
            raise MemoryError("omTensorCreate failed")
        return Tensor(h, obj, True, True)

    @property
    def __cuda_array_interface__(self):
        """Device tensors can be handed to torch / cupy without a copy
        (torch.as_tensor(t, device="cuda")); the Tensor must outlive the view."""
        if not self.device:
            raise AttributeError("host tensor")
        return {"shape": self.shape, "typestr": np.dtype(self.dtype).str,
                "data": (int(self.data_ptr or 0), False), "version": 2, "strides": None}

    @staticmethod
    def from_numpy(a):
        a = _c(a)
        shape = (ctypes.c_int64 * max(a.ndim, 1))(*a.shape)
        h = lib().omTensorCreate(a.ctypes.data, shape, a.ndim, _NP2OM[a.dtype])
        if not h:
            raise MemoryError("omTensorCreate failed")
        return Tensor(h, a)

    @staticmethod
    def empty(shape, dtype):
        return Tensor.from_numpy(np.empty(shape, dtype=dtype))

    @staticmethod
    def device_empty(shape, dtype):
        shape = tuple(int(s) for s in shape)
        cs = (ctypes.c_int64 * max(len(shape), 1))(*shape)
        h = lib().omcudaTensorCreateOnDevice(cs, len(shape),
                                             _NP2OM[np.dtype(dtype)])
        if not h:
            check()
            raise MemoryError("omcudaTensorCreateOnDevice failed")
        return Tensor(h, None, True)

    def to_device(self):
        h = lib().omcudaTensorToDevice(self.handle)
        if not h:
            check()
            raise MemoryError("omcudaTensorToDevice failed")
        return Tensor(h, None, True)

    @property
    def shape(self):
        L = lib()
        r = L.omTensorGetRank(self.handle)
        s = L.omTensorGetShape(self.handle)
        return tuple(int(s[i]) for i in range(r))

    @property
    def dtype(self):
        return _OM2NP[lib().omTensorGetDataType(self.handle)]

    @property
    def data_ptr(self):
        return lib().omTensorGetDataPtr(self.handle)

    def numpy(self):
        if not self.device:
            return self.array
        L = lib()
        h = L.omcudaTensorToHost(self.handle)
        if not h:
            check()
            raise MemoryError("omcudaTensorToHost failed")
        n = L.omTensorGetBufferSize(h)
        buf = (ctypes.c_char * max(n, 1)).from_address(L.omTensorGetDataPtr(h))
        out = np.frombuffer(buf, dtype=self.dtype, count=int(
            L.omTensorGetNumElems(h))).reshape(self.shape).copy()
        L.omTensorDestroy(h)
        return out

    def free(self):
        if self.handle:
            if self.device and not self.borrowed:
                lib().omcudaTensorDestroy(self.handle)
            else:
                lib().omTensorDestroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _h(t):
    return t.handle if t is not None else None


def _wrap(x, device):
    """numpy array / Tensor / None -> Tensor on the requested side."""
    if x is None or isinstance(x, Tensor):
        return x
    if hasattr(x, "__cuda_array_interface__"):
        return Tensor.from_cuda_array(x)
    t = Tensor.from_numpy(np.asarray(x))
    return t.to_device() if device else t


def _out(shape, dtype, device):
    return (Tensor.device_empty(shape, dtype) if device
            else Tensor.empty(shape, dtype))


# ---- op wrappers: numpy in, numpy out (host tensors staged inside the call),
# ---- or device=True to keep everything resident and get Tensors back.

def dynamic_quantize_linear(x, device=False):
    x = _wrap(x, device)
    y = _out(x.shape, np.uint8, device)
    s = _out((), np.float32, device)
    z = _out((), np.uint8, device)
    lib().omcudaDynamicQuantizeLinear(y.handle, s.handle, z.handle, x.handle)
    check()
    return (y, s, z) if device else (y.numpy(), s.numpy(), z.numpy())


def quantize_linear(x, scale, zp=None, out_dtype=np.uint8, device=False):
    x = _wrap(x, device)
    scale = _wrap(np.asarray(scale, np.float32), device)
    zp = _wrap(zp, device)
    y = _out(x.shape, out_dtype, device)
    lib().omcudaQuantizeLinear(y.handle, x.handle, scale.handle, _h(zp))
    check()
    return y if device else y.numpy()


def dequantize_linear(x, scale, zp=None, device=False):
    x = _wrap(x, device)
    scale = _wrap(np.asarray(scale, np.float32), device)
    zp = _wrap(zp, device)
    y = _out(x.shape, np.float32, device)
    lib().omcudaDequantizeLinear(y.handle, x.handle, scale.handle, _h(zp))
    check()
    return y if device else y.numpy()


def _matmul_shape(a_shape, b_shape):
    if len(b_shape) == 1:
        return tuple(a_shape[:-1])
    if len(a_shape) == 1:
        return tuple(b_shape[:-2]) + (b_shape[-1],)
    if len(b_shape) <= 2:
        return tuple(a_shape[:-1]) + (b_shape[-1],)
    try:
        batch = np.broadcast_shapes(tuple(a_shape[:-2]), tuple(b_shape[:-2]))
    except ValueError:  # let the library report the mismatch
        batch = tuple(a_shape[:-2])
    return tuple(batch) + (a_shape[-2], b_shape[-1])


def matmul_integer(A, B, a_zp=None, b_zp=None, device=False):
    A, B = _wrap(A, device), _wrap(B, device)
    a_zp, b_zp = _wrap(a_zp, device), _wrap(b_zp, device)
    Y = _out(_matmul_shape(A.shape, B.shape), np.int32, device)
    lib().omcudaMatMulInteger(Y.handle, A.handle, B.handle, _h(a_zp), _h(b_zp))
    check()
    return Y if device else Y.numpy()


def qlinear_matmul(a, a_scale, a_zp, b, b_scale, b_zp, y_scale, y_zp,
                   device=False):
    a, b = _wrap(a, device), _wrap(b, device)
    ts = [_wrap(np.asarray(v), device) if not isinstance(v, Tensor) else v
          for v in (a_scale, a_zp, b_scale, b_zp, y_scale, y_zp)]
    ydt = ts[5].dtype
    y = _out(_matmul_shape(a.shape, b.shape), ydt, device)
    lib().omcudaQLinearMatMul(y.handle, a.handle, ts[0].handle, ts[1].handle,
                              b.handle, ts[2].handle, ts[3].handle,
                              ts[4].handle, ts[5].handle)
    check()
    return y if device else y.numpy()


def dyn_quant_linear(X, Wq, w_scale, w_zp=None, bias=None, scale_form=0,
                     device=False):
    X, Wq = _wrap(X, device), _wrap(Wq, device)
    w_scale = _wrap(np.asarray(w_scale, np.float32)
                    if not isinstance(w_scale, Tensor) else w_scale, device)
    w_zp, bias = _wrap(w_zp, device), _wrap(bias, device)
    Y = _out(tuple(X.shape[:-1]) + (Wq.shape[-1],), np.float32, device)
    lib().omcudaDynQuantLinear(Y.handle, X.handle, Wq.handle, w_scale.handle,
                               _h(w_zp), _h(bias), scale_form)
    check()
    return Y if device else Y.numpy()


def softmax(x, axis=-1, device=False):
    x = _wrap(x, device)
    y = _out(x.shape, np.float32, device)
    lib().omcudaSoftmax(y.handle, x.handle, axis)
    check()
    return y if device else y.numpy()


def layer_normalization(x, gamma, beta=None, axis=-1, epsilon=1e-5,
                        device=False):
    x, gamma, beta = _wrap(x, device), _wrap(gamma, device), _wrap(beta, device)
    y = _out(x.shape, np.float32, device)
    lib().omcudaLayerNormalization(y.handle, x.handle, gamma.handle, _h(beta),
                                   axis, float(epsilon))
    check()
    return y if device else y.numpy()


def gelu(x, device=False):
    x = _wrap(x, device)
    y = _out(x.shape, np.float32, device)
    lib().omcudaGelu(y.handle, x.handle)
    check()
    return y if device else y.numpy()


def add(a, b, device=False):
    a, b = _wrap(a, device), _wrap(b, device)
    y = _out(a.shape, np.float32, device)
    lib().omcudaAdd(y.handle, a.handle, b.handle)
    check()
    return y if device else y.numpy()


def transpose_0213(x, device=False):
    x = _wrap(x, device)
    s = x.shape
    y = _out((s[0], s[2], s[1], s[3]), np.float32, device)
    lib().omcudaTranspose0213(y.handle, x.handle)
    check()
    return y if device else y.numpy()


def matmul_f32(a, b, device=False):
    a, b = _wrap(a, device), _wrap(b, device)
    y = _out(_matmul_shape(a.shape, b.shape), np.float32, device)
    lib().omcudaMatMulF32(y.handle, a.handle, b.handle)
    check()
    return y if device else y.numpy()


def attention(q, k, v, heads, scale, device=False):
    q, k, v = _wrap(q, device), _wrap(k, device), _wrap(v, device)
    y = _out(q.shape, np.float32, device)
    lib().omcudaAttention(y.handle, q.handle, k.handle, v.handle, heads,
                          float(scale))
    check()
    return y if device else y.numpy()


# ---- encoder model harness ---------------------------------------------------

class _EncoderConfig(ctypes.Structure):
    _fields_ = [("layers", ctypes.c_int64), ("hidden", ctypes.c_int64),
                ("heads", ctypes.c_int64), ("ffn", ctypes.c_int64),
                ("epsilon", ctypes.c_double)]


class _EncoderLayerWeights(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("wq", "wk", "wv", "wo", "w1", "w2")] +
                [("w_scale", ctypes.c_float * 6)] +
                [(n, ctypes.c_void_p) for n in ("bq", "bk", "bv", "bo", "b1", "b2",
                                                "ln1_gamma", "ln1_beta",
                                                "ln2_gamma", "ln2_beta")])


class Encoder:
    """The run_main_graph-shaped harness for the BERT-shaped encoder configs
    (omcudaEncoder* in omcuda.h).  `layers` is a list of dicts with int8
    weights wq,wk,wv,wo [H,H], w1 [H,F], w2 [F,H], `sc` (6 weight scales),
    f32 biases bq,bk,bv,bo,b1,b2 and ln1g,ln1b,ln2g,ln2b."""

    def __init__(self, hidden, heads, ffn, layers, epsilon=1e-5):
        L = lib()
        L.omcudaEncoderCreate.restype = ctypes.c_void_p
        L.omcudaEncoderCreate.argtypes = [ctypes.POINTER(_EncoderConfig)]
        L.omcudaEncoderSetLayer.argtypes = [ctypes.c_void_p, ctypes.c_int64,
                                            ctypes.POINTER(_EncoderLayerWeights)]
        L.omcudaEncoderRun.restype = ctypes.c_void_p
        L.omcudaEncoderRun.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        L.omcudaEncoderRunDev.argtypes = [ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_int64, ctypes.c_int64,
                                          ctypes.c_void_p, ctypes.c_void_p]
        L.omcudaEncoderDestroy.argtypes = [ctypes.c_void_p]
        cfg = _EncoderConfig(len(layers), hidden, heads, ffn, epsilon)
        self.hidden = hidden
        self.handle = L.omcudaEncoderCreate(ctypes.byref(cfg))
        if not self.handle:
            check()
            raise OmcudaError(EINVAL, "omcudaEncoderCreate failed")
        for i, w in enumerate(layers):
            keep = {}
            lw = _EncoderLayerWeights()
            names = {"wq": "wq", "wk": "wk", "wv": "wv", "wo": "wo", "w1": "w1",
                     "w2": "w2", "bq": "bq", "bk": "bk", "bv": "bv", "bo": "bo",
                     "b1": "b1", "b2": "b2", "ln1g": "ln1_gamma",
                     "ln1b": "ln1_beta", "ln2g": "ln2_gamma", "ln2b": "ln2_beta"}
            for src, dst in names.items():
                if w.get(src) is None:
                    continue
                keep[src] = Tensor.from_numpy(w[src])
                setattr(lw, dst, keep[src].handle)
            for j in range(6):
                lw.w_scale[j] = float(w["sc"][j])
            rc = L.omcudaEncoderSetLayer(self.handle, i, ctypes.byref(lw))
            if rc != 0:
                check()
                raise OmcudaError(rc, "omcudaEncoderSetLayer failed")

    def run(self, x):
        """run_main_graph: numpy [B,S,H] in, numpy out (staged through HBM), or
        a device Tensor in, device Tensor out."""
        L = lib()
        dev = isinstance(x, Tensor)
        t = x if dev else Tensor.from_numpy(np.asarray(x, np.float32))
        arr = (ctypes.c_void_p * 1)(t.handle)
        ins = L.omTensorListCreate(arr, 1)
        outs = L.omcudaEncoderRun(self.handle, ins)
        L.omTensorListDestroyShallow(ins)
        if not outs:
            check()
            raise OmcudaError(ECUDA, "omcudaEncoderRun returned NULL")
        o = L.omTensorListGetOmtByIndex(outs, 0)
        L.omTensorListDestroyShallow(outs)
        if dev:
            return Tensor(o, None, True)
        n = L.omTensorGetNumElems(o)
        buf = (ctypes.c_char * (4 * n)).from_address(L.omTensorGetDataPtr(o))
        out = np.frombuffer(buf, dtype=np.float32, count=n).reshape(t.shape).copy()
        L.omTensorDestroy(o)
        return out

    def run_into(self, x, y):
        """run_main_graph with the caller's output: x, y are Tensors (host or
        device) of shape [B,S,H]; y is filled in place."""
        L = lib()
        L.omcudaEncoderRunInto.argtypes = [ctypes.c_void_p] * 3
        rc = L.omcudaEncoderRunInto(self.handle, y.handle, x.handle)
        if rc != 0:
            check()
            raise OmcudaError(rc, "omcudaEncoderRunInto failed")

    def submit(self, x, y):
        """Pipelined run_into for host Tensors: queues copy-in, run, copy-out
        and returns; y is complete after wait()."""
        L = lib()
        L.omcudaEncoderSubmit.argtypes = [ctypes.c_void_p] * 3
        rc = L.omcudaEncoderSubmit(self.handle, y.handle, x.handle)
        if rc != 0:
            check()
            raise OmcudaError(rc, "omcudaEncoderSubmit failed")

    def wait(self):
        L = lib()
        L.omcudaEncoderWait.argtypes = [ctypes.c_void_p]
        rc = L.omcudaEncoderWait(self.handle)
        if rc != 0:
            check()
            raise OmcudaError(rc, "omcudaEncoderWait failed")

    def run_dev(self, x_ptr, batch, seq, y_ptr, stream):
        rc = lib().omcudaEncoderRunDev(self.handle, x_ptr, batch, seq, y_ptr, stream)
        if rc != 0:
            check()
            raise OmcudaError(rc, "omcudaEncoderRunDev failed")

    def run_tapped(self, x):
        """Runs numpy x [B,S,H] with the parity-test tap on (omcudaEncoderSetTap)
        and returns (y, taps): taps[l] maps x, xq_x, ctx, xq_ctx, h1, xq_h1, f,
        xq_f, y to numpy arrays of layer l, and taps[l]["sites"] lists, for the
        four quantize sites x, ctx, h1, f, the (scale, zero point) the library
        derived, as (np.float32, np.uint8)."""
        L = lib()
        L.omcudaEncoderGetTapLayout.argtypes = [ctypes.c_void_p, ctypes.c_int64,
                                                ctypes.c_int64, ctypes.c_void_p]
        L.omcudaEncoderSetTap.argtypes = [ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_int64]
        x = _c(x, np.float32)
        B, S, H = x.shape
        lay = (ctypes.c_int64 * 12)()
        rc = L.omcudaEncoderGetTapLayout(self.handle, B, S, lay)
        if rc != 0:
            check()
        names = ("x", "xq_x", "ctx", "xq_ctx", "h1", "xq_h1", "f", "xq_f", "y")
        off = dict(zip(names, lay[:9]))
        stride, p_off, total = lay[9], lay[10], lay[11]
        buf = Tensor.device_empty((total,), np.uint8)
        rc = L.omcudaEncoderSetTap(self.handle, buf.data_ptr, total)
        if rc != 0:
            check()
        try:
            y = self.run(x)
        finally:
            L.omcudaEncoderSetTap(self.handle, None, 0)
        raw = buf.numpy()
        buf.free()
        T = B * S
        nl = (p_off // stride) if stride else 0
        F = (off["xq_f"] - off["f"]) // (4 * T)
        params = raw[p_off:p_off + (4 * nl + 1) * 16]
        taps = []
        for l in range(nl):
            d = {}
            for n in names:
                cols = F if n in ("f", "xq_f") else H
                dt, esz = (np.uint8, 1) if n.startswith("xq") else (np.float32, 4)
                a = l * stride + off[n]
                d[n] = raw[a:a + T * cols * esz].view(dt).reshape(T, cols)
            sites = []
            for k in range(4):
                slot = params[(4 * l + k) * 16:(4 * l + k + 1) * 16]
                sites.append((slot[8:12].view(np.float32)[0], slot[12]))
            d["sites"] = sites
            taps.append(d)
        return y, taps

    def set_range_sync(self, fn):
        """fn: an omcuda.sharding.make_range_sync(...) callback, or None for
        per-shard quantization ranges (the default)."""
        L = lib()
        L.omcudaEncoderSetRangeSync.argtypes = [ctypes.c_void_p, ctypes.c_void_p,
                                                ctypes.c_void_p]
        self._range_sync = fn            # keeps the ctypes callback alive
        ptr = ctypes.cast(fn, ctypes.c_void_p) if fn is not None else None
        if L.omcudaEncoderSetRangeSync(self.handle, ptr, None) != 0:
            check()

    def set_profiling(self, on):
        lib().omcudaEncoderSetProfiling.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib().omcudaEncoderSetProfiling(self.handle, int(on))

    def gemm_stats(self):
        """(summed GEMM ms, summed 2*M*N*K, launches) since profiling began."""
        L = lib()
        L.omcudaEncoderGemmStats.argtypes = [ctypes.c_void_p] * 4
        ms, ops, n = ctypes.c_double(), ctypes.c_double(), ctypes.c_int64()
        rc = L.omcudaEncoderGemmStats(self.handle, ctypes.byref(ms),
                                      ctypes.byref(ops), ctypes.byref(n))
        if rc != 0:
            check()
        return ms.value, ops.value, n.value

    def close(self):
        if self.handle:
            lib().omcudaEncoderDestroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

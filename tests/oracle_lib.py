"""ctypes wrapper of the CPU oracle (oracle/oracle.c).  Test infrastructure:
imported by tests, the smoke check and the benchmark's CPU-baseline leg only."""
import ctypes

import numpy as np

_f32p = ctypes.POINTER(ctypes.c_float)
_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int


def _c(a, dtype=None):
    """C-contiguous view/copy that keeps rank-0 arrays rank 0."""
    return np.require(a, dtype=dtype, requirements="C")


def _p(a):
    return a.ctypes.data_as(_vp) if a is not None else None


class EncoderWeights(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ("wq", "wk", "wv", "wo", "w1", "w2")] + \
               [("sc", ctypes.c_float * 6)] + \
               [(n, _vp) for n in ("bq", "bk", "bv", "bo", "b1", "b2",
                                   "ln1g", "ln1b", "ln2g", "ln2b")]


class Oracle:
    def __init__(self, path):
        self.L = ctypes.CDLL(path)
        L = self.L
        L.orc_round_even.restype = ctypes.c_float
        L.orc_round_even.argtypes = [ctypes.c_float]
        L.orc_selftest_round_even_exhaustive.restype = _i64
        L.orc_max_threads.restype = _i32
        L.orc_set_quant_mode.argtypes = [_i32]
        L.orc_dql_params.argtypes = [ctypes.c_float, ctypes.c_float, _vp, _vp, _vp]
        L.orc_minmax_f32.argtypes = [_vp, _i64, _vp, _vp]
        L.orc_quantize_u8.argtypes = [_vp, _i64, ctypes.c_float, ctypes.c_float, _vp]
        L.orc_quantize_i8.argtypes = [_vp, _i64, ctypes.c_float, ctypes.c_float, _vp]
        L.orc_dynamic_quantize_linear.argtypes = [_vp, _i64, _vp, _vp, _vp]
        L.orc_matmul_integer.argtypes = [_vp, _i32, _vp, _i32, _i64, _i64, _i64,
                                         _vp, _i64, _vp, _i64, _vp]
        L.orc_qlinear_matmul.argtypes = [_vp, _i32, ctypes.c_float, ctypes.c_int32,
                                         _vp, _i32, _vp, _vp, _i64, ctypes.c_float,
                                         ctypes.c_int32, _i32, _i64, _i64, _i64, _vp]
        L.orc_dequant_tail.argtypes = [_vp, _i64, _i64, ctypes.c_float,
                                       ctypes.c_float, _i32, _vp, _vp]
        L.orc_dequantize_linear.argtypes = [_vp, _i32, _i64, ctypes.c_float,
                                            ctypes.c_int32, _vp]
        L.orc_softmax_lastdim.argtypes = [_vp, _i64, _i64, _vp]
        L.orc_layernorm.argtypes = [_vp, _i64, _i64, _vp, _vp, ctypes.c_float, _vp]
        L.orc_gelu.argtypes = [_vp, _i64, _vp]
        L.orc_add.argtypes = [_vp, _vp, _i64, _vp]
        L.orc_transpose_0213.argtypes = [_vp, _i64, _i64, _i64, _i64, _vp]
        L.orc_matmul_f32.argtypes = [_vp, _vp, _i64, _i64, _i64, _i64, _vp]
        L.orc_attention.argtypes = [_vp, _vp, _vp, _i64, _i64, _i64, _i64,
                                    ctypes.c_float, _vp]
        L.orc_dyn_quant_linear.argtypes = [_vp, _i64, _i64, _vp, _i64,
                                           ctypes.c_float, _vp, _vp, _vp, _vp,
                                           _vp, _vp]
        L.orc_encoder_layer.argtypes = [_vp, _i64, _i64, _i64, _i64, _i64,
                                        ctypes.POINTER(EncoderWeights),
                                        ctypes.c_float, _vp]
        L.orc_ref_shaped_matmul_integer.argtypes = [_vp, _vp, _i64, _i64, _i64,
                                                    ctypes.c_int32, _vp, _i32]

    # -- scalar --
    def round_even(self, x):
        return float(self.L.orc_round_even(np.float32(x)))

    def dql_params(self, mn, mx):
        s = np.zeros((), np.float32)
        zf = np.zeros((), np.float32)
        z = np.zeros((), np.uint8)
        self.L.orc_dql_params(np.float32(mn), np.float32(mx), _p(s), _p(zf), _p(z))
        return s, zf, z

    # -- quantization --
    def dynamic_quantize_linear(self, x):
        x = _c(x, np.float32)
        y = np.empty(x.shape, np.uint8)
        s = np.zeros((), np.float32)
        z = np.zeros((), np.uint8)
        self.L.orc_dynamic_quantize_linear(_p(x), x.size, _p(y), _p(s), _p(z))
        return y, s, z

    def quantize(self, x, scale, zp, signed=False):
        x = _c(x, np.float32)
        y = np.empty(x.shape, np.int8 if signed else np.uint8)
        fn = self.L.orc_quantize_i8 if signed else self.L.orc_quantize_u8
        fn(_p(x), x.size, np.float32(scale), np.float32(zp), _p(y))
        return y

    def dequantize_linear(self, x, scale, zp=0):
        x = _c(x)
        code = {np.dtype(np.uint8): 0, np.dtype(np.int8): 1,
                np.dtype(np.int32): 2}[x.dtype]
        y = np.empty(x.shape, np.float32)
        self.L.orc_dequantize_linear(_p(x), code, x.size, np.float32(scale),
                                     int(zp), _p(y))
        return y

    # -- matmuls --
    def matmul_integer_2d(self, A, B, a_zp=None, b_zp=None):
        A = _c(A)
        B = _c(B)
        M, K = A.shape
        K2, N = B.shape
        assert K == K2
        Y = np.empty((M, N), np.int32)
        az = None if a_zp is None else _c(a_zp, A.dtype).reshape(-1)
        bz = None if b_zp is None else _c(b_zp, B.dtype).reshape(-1)
        self.L.orc_matmul_integer(
            _p(A), int(A.dtype == np.int8), _p(B), int(B.dtype == np.int8), M, N, K,
            _p(az), 0 if az is None else az.size, _p(bz),
            0 if bz is None else bz.size, _p(Y))
        return Y

    def matmul_integer(self, A, B, a_zp=None, b_zp=None):
        """numpy-matmul broadcasting over the 2-D oracle."""
        A = np.asarray(A)
        B = np.asarray(B)
        a1, b1 = A.ndim == 1, B.ndim == 1
        A2 = A[None, :] if a1 else A
        B2 = B[:, None] if b1 else B
        bshape = np.broadcast_shapes(A2.shape[:-2], B2.shape[:-2])
        Ab = np.broadcast_to(A2, bshape + A2.shape[-2:])
        Bb = np.broadcast_to(B2, bshape + B2.shape[-2:])
        out = np.empty(bshape + (A2.shape[-2], B2.shape[-1]), np.int32)
        for idx in np.ndindex(*bshape):
            out[idx] = self.matmul_integer_2d(Ab[idx], Bb[idx], a_zp, b_zp)
        if a1:
            out = out[..., 0, :]
        if b1:
            out = out[..., 0]
        return out

    def qlinear_matmul(self, A, a_scale, a_zp, B, b_scale, b_zp, y_scale, y_zp):
        A = _c(A)
        B = _c(B)
        lead = A.shape[:-1]
        K = A.shape[-1]
        A2 = A.reshape(-1, K)
        M = A2.shape[0]
        N = B.shape[1]
        b_scale = _c(b_scale, np.float32).reshape(-1)
        b_zp = _c(b_zp, B.dtype).reshape(-1)
        if b_zp.size != b_scale.size:
            n = max(b_zp.size, b_scale.size)
            b_zp = _c(np.broadcast_to(b_zp, (n,)))
            b_scale = _c(np.broadcast_to(b_scale, (n,)))
        y_zp = np.asarray(y_zp)
        Y = np.empty((M, N), y_zp.dtype)
        self.L.orc_qlinear_matmul(
            _p(A2), int(A.dtype == np.int8), np.float32(a_scale), int(a_zp),
            _p(B), int(B.dtype == np.int8), _p(b_scale), _p(b_zp), b_scale.size,
            np.float32(y_scale), int(y_zp), int(y_zp.dtype == np.int8), M, N, K,
            _p(Y))
        return Y.reshape(lead + (N,))

    def dequant_tail(self, acc, s0, s1=0.0, form=0, bias=None):
        acc = _c(acc, np.int32)
        M, N = acc.reshape(-1, acc.shape[-1]).shape
        y = np.empty(acc.shape, np.float32)
        b = None if bias is None else _c(bias, np.float32)
        self.L.orc_dequant_tail(_p(acc), M, N, np.float32(s0), np.float32(s1),
                                form, _p(b), _p(y))
        return y

    def dyn_quant_linear(self, X, W, w_scale, bias=None):
        X = _c(X, np.float32)
        W = _c(W, np.int8)
        K, N = W.shape
        X2 = X.reshape(-1, K)
        M = X2.shape[0]
        Y = np.empty((M, N), np.float32)
        xq = np.empty((M, K), np.uint8)
        acc = np.empty((M, N), np.int32)
        s = np.zeros((), np.float32)
        z = np.zeros((), np.uint8)
        b = None if bias is None else _c(bias, np.float32)
        self.L.orc_dyn_quant_linear(_p(X2), M, K, _p(W), N, np.float32(w_scale),
                                    _p(b), _p(Y), _p(xq), _p(s), _p(z), _p(acc))
        return {"Y": Y.reshape(X.shape[:-1] + (N,)), "xq": xq.reshape(X.shape),
                "x_scale": s, "x_zp": z, "acc": acc.reshape(X.shape[:-1] + (N,))}

    # -- fp32 ops --
    def softmax(self, x):
        x = _c(x, np.float32)
        y = np.empty_like(x)
        self.L.orc_softmax_lastdim(_p(x), x.size // x.shape[-1], x.shape[-1], _p(y))
        return y

    def layernorm(self, x, gamma, beta, eps=1e-5):
        x = _c(x, np.float32)
        y = np.empty_like(x)
        g = _c(gamma, np.float32)
        b = None if beta is None else _c(beta, np.float32)
        self.L.orc_layernorm(_p(x), x.size // x.shape[-1], x.shape[-1], _p(g),
                             _p(b), np.float32(eps), _p(y))
        return y

    def gelu(self, x):
        x = _c(x, np.float32)
        y = np.empty_like(x)
        self.L.orc_gelu(_p(x), x.size, _p(y))
        return y

    def transpose_0213(self, x):
        x = _c(x, np.float32)
        B, S, H, D = x.shape
        y = np.empty((B, H, S, D), np.float32)
        self.L.orc_transpose_0213(_p(x), B, S, H, D, _p(y))
        return y

    def matmul_f32(self, A, B):
        A = _c(A, np.float32)
        B = _c(B, np.float32)
        batch = int(np.prod(A.shape[:-2])) if A.ndim > 2 else 1
        M, K = A.shape[-2:]
        N = B.shape[-1]
        C = np.empty(A.shape[:-1] + (N,), np.float32)
        self.L.orc_matmul_f32(_p(A), _p(B), batch, M, N, K, _p(C))
        return C

    def attention(self, q, k, v, heads, scale):
        q = _c(q, np.float32)
        k = _c(k, np.float32)
        v = _c(v, np.float32)
        B, S, H = q.shape
        out = np.empty_like(q)
        self.L.orc_attention(_p(q), _p(k), _p(v), B, S, heads, H // heads,
                             np.float32(scale), _p(out))
        return out

    def encoder_layer(self, x, B, S, H, heads, F, w, eps=1e-5):
        """w: dict with wq,wk,wv,wo,w1,w2 (int8), sc (6 floats), biases, ln."""
        x = _c(x, np.float32)
        keep = {k: _c(v) for k, v in w.items() if k != "sc"}
        ew = EncoderWeights()
        for name in ("wq", "wk", "wv", "wo", "w1", "w2", "bq", "bk", "bv", "bo",
                     "b1", "b2", "ln1g", "ln1b", "ln2g", "ln2b"):
            setattr(ew, name, keep[name].ctypes.data)
        for i in range(6):
            ew.sc[i] = float(w["sc"][i])
        y = np.empty_like(x)
        self.L.orc_encoder_layer(_p(x), B, S, H, heads, F, ctypes.byref(ew),
                                 np.float32(eps), _p(y))
        return y

    def ref_shaped_matmul_integer(self, A, B, a_zp, threads=1):
        A = _c(A, np.uint8)
        B = _c(B, np.int8)
        M, K = A.shape
        N = B.shape[1]
        Y = np.empty((M, N), np.int32)
        self.L.orc_ref_shaped_matmul_integer(_p(A), _p(B), M, N, K, int(a_zp),
                                             _p(Y), threads)
        return Y

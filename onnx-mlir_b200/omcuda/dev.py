"""ctypes binding of libomcuda's device-pointer entry points (omcudaDev*).

For callers that already hold device buffers and a CUDA stream: the benchmark
(torch tensors supply the memory and the stream) and tests that pick a kernel
explicitly.  Pointers are plain integers (`tensor.data_ptr()`)."""
import ctypes

from . import OmcudaError, check, lib

EPI_I32, EPI_DEQUANT, EPI_REQUANT, EPI_DEQUANT_SPLIT = 0, 1, 2, 3
EPI_DEQUANT_RANGE, EPI_DEQUANT_QUANT = 4, 5
KERNEL_AUTO, KERNEL_TENSOR_CORE, KERNEL_SIMT = 0, 1, 2

_vp, _i64, _i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int


class PreparedB(ctypes.Structure):
    _fields_ = [("bt", _vp), ("colsum", _vp), ("K", _i64), ("N", _i64),
                ("kp", _i64), ("b_signed", _i32)]


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("M", _i64), ("N", _i64), ("K", _i64),
        ("A", _vp), ("a_signed", _i32),
        ("B", PreparedB),
        ("a_zp", _vp), ("a_zp_len", _i64),
        ("b_zp", _vp), ("b_zp_len", _i64),
        ("a_rowsum", _vp),
        ("epilogue", _i32),
        ("Y", _vp),
        ("sa", _vp), ("sb", _vp), ("sb_len", _i64),
        ("scale_form", _i32),
        ("bias", _vp),
        ("gelu", _i32),
        ("y_zp", ctypes.c_int32),
        ("y_signed", _i32),
        ("out_minmax", _vp),
        ("kernel_choice", _i32),
        ("residual", _vp),
        ("q_range", _vp), ("q_params", _vp), ("q_scale", _vp), ("q_zp", _vp),
    ]


_bound = False


def _bind():
    global _bound
    L = lib()
    if _bound:
        return L
    L.omcudaDevDqlScratchBytes.restype = _i64
    L.omcudaDevDqlScratchBytes.argtypes = [_i64]
    L.omcudaDevDynamicQuantizeLinear.argtypes = [_vp, _i64, _vp, _vp, _vp, _vp, _vp]
    L.omcudaDevQuantizeLinear.argtypes = [_vp, _i64, _vp, _i32, _vp, _vp, _vp]
    L.omcudaDevPreparedBBytes.restype = _i64
    L.omcudaDevPreparedBBytes.argtypes = [_i64, _i64, ctypes.POINTER(_i64)]
    L.omcudaDevPrepareB.argtypes = [_vp, _i32, _i64, _i64,
                                    ctypes.POINTER(PreparedB), _vp]
    L.omcudaDevGemmI8.argtypes = [ctypes.POINTER(GemmArgs), _vp]
    L.omcudaDevRequantScale.argtypes = [_vp, _vp, _i64, _vp, _vp, _vp]
    L.omcudaDevRowSum.argtypes = [_vp, _i32, _i64, _i64, _vp, _vp]
    L.omcudaDevDequantizeLinear.argtypes = [_vp, _i32, _i64, _vp, _vp, _vp, _vp]
    L.omcudaDevSoftmax.argtypes = [_vp, _i64, _i64, _vp, _vp]
    L.omcudaDevLayerNorm.argtypes = [_vp, _vp, _i64, _i64, _vp, _vp,
                                     ctypes.c_float, _vp, _vp, _vp]
    L.omcudaDevGelu.argtypes = [_vp, _i64, _vp, _vp]
    L.omcudaDevAdd.argtypes = [_vp, _vp, _i64, _vp, _vp]
    L.omcudaDevTranspose0213.argtypes = [_vp, _i64, _i64, _i64, _i64, _vp, _vp]
    L.omcudaDevMatMulF32.argtypes = [_vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp]
    L.omcudaDevAttention.argtypes = [_vp, _vp, _vp, _i64, _i64, _i64, _i64,
                                     ctypes.c_float, _vp, _vp]
    L.omcudaDevSplitBf16.argtypes = [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _vp]
    L.omcudaDevAttentionBf16Supported.argtypes = [_i64] * 6
    L.omcudaDevAttentionBf16.argtypes = [_vp, _vp] + [_i64] * 8 + [
        ctypes.c_float, _vp, _i64, _vp, _vp]
    L.omcudaDevSetWaitLimitNs.argtypes = [_i64]
    L.omcudaDevSetWaitLimitNs.restype = None
    L.omcudaDevSelfTestBoundedWait.argtypes = [_vp, _vp]
    _bound = True
    return L


def _ok(rc):
    if rc != 0:
        check()
        raise OmcudaError(rc, "device entry point failed")


def dql_scratch_bytes(n=0):
    return int(_bind().omcudaDevDqlScratchBytes(n))


def dynamic_quantize_linear(x, n, y, y_scale, y_zp, scratch, stream):
    _ok(_bind().omcudaDevDynamicQuantizeLinear(x, n, y, y_scale, y_zp, scratch,
                                               stream))


def prepared_b_bytes(K, N):
    kp = _i64()
    nbytes = _bind().omcudaDevPreparedBBytes(K, N, ctypes.byref(kp))
    return int(nbytes), int(kp.value)


def prepare_b(B, b_signed, K, N, bt, colsum, stream):
    pb = PreparedB()
    pb.bt, pb.colsum = bt, colsum
    _ok(_bind().omcudaDevPrepareB(B, int(b_signed), K, N, ctypes.byref(pb),
                                  stream))
    return pb


def gemm_i8(args, stream):
    _ok(_bind().omcudaDevGemmI8(ctypes.byref(args), stream))


def range_init(ranges, count, stream):
    L = _bind()
    L.omcudaDevRangeInit.argtypes = [_vp, _i64, _vp]
    _ok(L.omcudaDevRangeInit(ranges, count, stream))


def quantize_from_range(x, n, rng, y, params, y_scale, y_zp, stream):
    L = _bind()
    L.omcudaDevQuantizeFromRange.argtypes = [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp]
    _ok(L.omcudaDevQuantizeFromRange(x, n, rng, y, params, y_scale, y_zp, stream))


def requant_scale(a_scale, b_scale, n, y_scale, S, stream):
    _ok(_bind().omcudaDevRequantScale(a_scale, b_scale, n, y_scale, S, stream))


def row_sum(A, a_signed, M, K, out, stream):
    _ok(_bind().omcudaDevRowSum(A, int(a_signed), M, K, out, stream))


def softmax(x, rows, cols, y, stream):
    _ok(_bind().omcudaDevSoftmax(x, rows, cols, y, stream))


def layernorm(x, residual, rows, cols, gamma, beta, eps, y, out_minmax, stream):
    _ok(_bind().omcudaDevLayerNorm(x, residual, rows, cols, gamma, beta, eps, y,
                                   out_minmax, stream))


def gelu(x, n, y, stream):
    _ok(_bind().omcudaDevGelu(x, n, y, stream))


def add(a, b, n, y, stream):
    _ok(_bind().omcudaDevAdd(a, b, n, y, stream))


def attention(q, k, v, B, S, heads, dh, scale, out, stream):
    _ok(_bind().omcudaDevAttention(q, k, v, B, S, heads, dh, scale, out, stream))


def split_bf16(x, rows, cols, ld_x, hi, lo, ld_planes, col0, stream):
    _ok(_bind().omcudaDevSplitBf16(x, rows, cols, ld_x, hi, lo, ld_planes, col0,
                                   stream))


def attention_bf16(hi, lo, ld_planes, q_col, k_col, v_col, B, S, heads, dh, scale,
                   out, ld_out, out_range, stream):
    _ok(_bind().omcudaDevAttentionBf16(hi, lo, ld_planes, q_col, k_col, v_col, B,
                                       S, heads, dh, scale, out, ld_out,
                                       out_range, stream))


def set_wait_limit_ns(ns):
    """Limit of every device-side wait of the tensor-core kernels (0: default)."""
    _bind().omcudaDevSetWaitLimitNs(int(ns))


def selftest_bounded_wait(waited_ns, stream):
    """Launches the one-CTA kernel that waits on a barrier nothing signals."""
    _ok(_bind().omcudaDevSelfTestBoundedWait(waited_ns, stream))

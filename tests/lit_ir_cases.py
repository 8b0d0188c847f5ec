"""Loads tests/golden/lit_ir_golden.json (vectors obtained by executing the Krnl
IR the reference's lowering tests expect) and maps each case onto a callable
backend: the CPU oracle or the CUDA library."""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = json.load(open(os.path.join(HERE, "golden", "lit_ir_golden.json")))["cases"]


MODE_CASES = json.load(open(os.path.join(HERE, "golden", "lit_ir_golden_modes.json")))["cases"]
MODE_FLAGS = {"no_zero_point": 1, "fast_math": 2}   # OMCUDA_MODE_* / ORC_MODE_*


def mode_case_id(c):
    return "%s-%s-%d" % (c["mode"], c["function"], len(c["inputs"][0]["data"]))


def _arr(t):
    return np.array(t["data"], dtype=np.dtype(t["dtype"])).reshape(t["shape"])


def case_id(c):
    return "%s-%d" % (c["function"], len(c["inputs"][0]["data"]))


def run_case(c, backend):
    """backend: object with dynamic_quantize_linear, quantize_linear,
    dequantize_linear, matmul_integer, qlinear_matmul taking numpy arrays.
    Returns (got_outputs, want_outputs)."""
    ins = [_arr(t) for t in c["inputs"]]
    want = [_arr(t) for t in c["outputs"]]
    fn = c["function"]
    if fn == "test_dynamic_quantize_linear":
        got = list(backend.dynamic_quantize_linear(ins[0]))
    elif fn.startswith("test_quantize_linear"):
        got = [backend.quantize_linear(ins[0], ins[1], ins[2], want[0].dtype)]
    elif fn.startswith("test_dequantizelinear"):
        got = [backend.dequantize_linear(ins[0], ins[1], ins[2])]
    elif fn.startswith("test_matmulinteger"):
        got = [backend.matmul_integer(ins[0], ins[1], ins[2], ins[3])]
    elif fn.startswith("qlinearmatmul"):
        got = [backend.qlinear_matmul(*ins)]
    else:
        raise KeyError(fn)
    return got, want


class OracleBackend:
    def __init__(self, orc):
        self.o = orc

    def dynamic_quantize_linear(self, x):
        return self.o.dynamic_quantize_linear(x)

    def quantize_linear(self, x, scale, zp, out_dtype):
        return self.o.quantize(x, float(scale.reshape(-1)[0]), float(zp.reshape(-1)[0]),
                               signed=(np.dtype(out_dtype) == np.int8)).reshape(x.shape)

    def dequantize_linear(self, x, scale, zp):
        return self.o.dequantize_linear(x, float(scale.reshape(-1)[0]), int(zp.reshape(-1)[0]))

    def matmul_integer(self, A, B, az, bz):
        return self.o.matmul_integer_2d(A, B, az, bz)

    def qlinear_matmul(self, a, a_s, a_z, b, b_s, b_z, y_s, y_z):
        return self.o.qlinear_matmul(a, float(a_s[0]), a_z[0], b, b_s, b_z, float(y_s[0]), y_z[0])


class GpuBackend:
    def __init__(self, m):
        self.m = m

    def dynamic_quantize_linear(self, x):
        return self.m.dynamic_quantize_linear(x)

    def quantize_linear(self, x, scale, zp, out_dtype):
        return self.m.quantize_linear(x, scale, zp, out_dtype=out_dtype)

    def dequantize_linear(self, x, scale, zp):
        return self.m.dequantize_linear(x, scale, zp)

    def matmul_integer(self, A, B, az, bz):
        return self.m.matmul_integer(A, B, az, bz)

    def qlinear_matmul(self, *a):
        return self.m.qlinear_matmul(*a)


def assert_same(got, want):
    assert len(got) == len(want)
    for g, w in zip(got, want):
        g = np.asarray(g)
        assert g.dtype == w.dtype, (g.dtype, w.dtype)
        assert g.reshape(-1).tobytes() == w.reshape(-1).tobytes(), (g.reshape(-1)[:8], w.reshape(-1)[:8])


# ---- fp32 ops of the encoder graphs (tests/golden/lit_ir_golden_fp32.json) ----------

import base64  # noqa: E402

FP32_CASES = json.load(open(os.path.join(HERE, "golden", "lit_ir_golden_fp32.json")))["cases"]


def _f32(t):
    return np.frombuffer(base64.b64decode(t["f32_le_b64"]), "<f4").reshape(t["shape"]).copy()


def fp32_case_id(c):
    return c["function"]


def run_fp32_case(c, backend):
    """backend: object with softmax (last axis), matmul_f32 (numpy matmul
    broadcasting), gelu and layernorm (last axis, [C] parameters, epsilon).
    Returns (got, want, kind) with kind in softmax / matmul / gelu / layernorm;
    for gelu also the input (its bound depends on it)."""
    ins = [_f32(t) for t in c["inputs"]]
    want = _f32(c["outputs"][0])
    fn = c["function"]
    if fn == "test_softmax_v13":          # axis = 1 of [10,20,30]
        x = np.ascontiguousarray(ins[0].transpose(0, 2, 1))
        return backend.softmax(x).transpose(0, 2, 1), want, "softmax", None
    if fn == "test_softmax_v11":          # opset 11: axis = 1 coerces to [10, 600]
        return backend.softmax(ins[0].reshape(10, 600)).reshape(want.shape), want, "softmax", None
    if fn.startswith("test_matmul"):
        return backend.matmul_f32(ins[0], ins[1]).reshape(want.shape), want, "matmul", None
    if fn == "test_gelu_none":
        return backend.gelu(ins[0]), want, "gelu", ins[0]
    if fn.startswith("layernorm"):        # axis = -2 of [2,64,31,3]: rows of 93
        x = ins[0].reshape(128, 93)
        got = backend.layernorm(x, ins[1].reshape(-1), ins[2].reshape(-1), 9.99999974e-6)
        return got.reshape(want.shape), want, "layernorm", None
    raise KeyError(fn)


class OracleFp32Backend:
    def __init__(self, orc):
        self.o = orc

    def softmax(self, x):
        return self.o.softmax(x)

    def matmul_f32(self, a, b):
        a1, b1 = a.ndim == 1, b.ndim == 1
        a2 = a[None, :] if a1 else a
        b2 = b[:, None] if b1 else b
        bs = np.broadcast_shapes(a2.shape[:-2], b2.shape[:-2])
        ab = np.ascontiguousarray(np.broadcast_to(a2, bs + a2.shape[-2:]))
        bb = np.ascontiguousarray(np.broadcast_to(b2, bs + b2.shape[-2:]))
        out = self.o.matmul_f32(ab, bb)
        if a1:
            out = out[..., 0, :]
        if b1:
            out = out[..., 0]
        return out

    def gelu(self, x):
        return self.o.gelu(x)

    def layernorm(self, x, g, b, eps):
        return self.o.layernorm(x, g, b, eps)


class GpuFp32Backend:
    def __init__(self, m):
        self.m = m

    def softmax(self, x):
        return self.m.softmax(x)

    def matmul_f32(self, a, b):
        return self.m.matmul_f32(a, b)

    def gelu(self, x):
        return self.m.gelu(x)

    def layernorm(self, x, g, b, eps):
        return self.m.layer_normalization(x, g, b, epsilon=eps)

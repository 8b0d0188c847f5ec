"""Loads tests/golden/lit_ir_golden.json (vectors obtained by executing the Krnl
IR the reference's lowering tests expect) and maps each case onto a callable
backend: the CPU oracle or the CUDA library."""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = json.load(open(os.path.join(HERE, "golden", "lit_ir_golden.json")))["cases"]


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

"""GPU parity against vectors obtained by executing the Krnl IR that the
reference's own lowering tests expect (tests/golden/lit_ir_golden.json):
DynamicQuantizeLinear, QuantizeLinear, DequantizeLinear, MatMulInteger (per
tensor and per row zero points) and QLinearMatMul (i8 and ui8), bit-exact."""
import pytest

import lit_ir_cases

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", lit_ir_cases.CASES, ids=lit_ir_cases.case_id)
def test_gpu_matches_executed_lit_ir(gpu, case):
    got, want = lit_ir_cases.run_case(case, lit_ir_cases.GpuBackend(gpu))
    lit_ir_cases.assert_same(got, want)


@pytest.mark.parametrize("case", lit_ir_cases.FP32_CASES, ids=lit_ir_cases.fp32_case_id)
def test_gpu_fp32_ops_match_executed_lit_ir(gpu, case):
    # The fp32 ops between the quantized linears against the executed IR of the
    # reference's Softmax / MatMul / Gelu / LayerNormalization lowering tests
    # (tests/golden/lit_ir_golden_fp32.json): 1e-3 relative where a reduction
    # is reordered, the Gelu bound of omcuda.h for Gelu.
    import numpy as np
    got, want, kind, x = lit_ir_cases.run_fp32_case(case, lit_ir_cases.GpuFp32Backend(gpu))
    assert got.shape == want.shape
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    if kind == "gelu":
        bound = 4e-6 * np.abs(want.astype(np.float64)) + \
            np.where(x < 0, 0.5 * np.abs(x.astype(np.float64)) * 2.0 ** -24, 0.0)
        assert (err <= bound).all(), (x[err > bound], got[err > bound], want[err > bound])
    else:
        scale = np.sqrt((want.astype(np.float64) ** 2).mean())
        assert (err <= 1e-3 * np.abs(want) + 1e-5 * scale).all(), err.max()


@pytest.mark.parametrize("case", lit_ir_cases.MODE_CASES, ids=lit_ir_cases.mode_case_id)
def test_gpu_modes_match_executed_lit_ir(gpu, case):
    # The reference's non-default arithmetic modes (omcudaSetQuantizationMode)
    # against the executed IR of its lowering tests for those options.
    L = gpu.lib()
    L.omcudaSetQuantizationMode(lit_ir_cases.MODE_FLAGS[case["mode"]])
    try:
        got, want = lit_ir_cases.run_case(case, lit_ir_cases.GpuBackend(gpu))
    finally:
        L.omcudaSetQuantizationMode(0)
    lit_ir_cases.assert_same(got, want)


@pytest.mark.parametrize("flags", [1, 2, 3])
def test_gpu_modes_on_large_tensors(gpu, orc, flags):
    # The vectorised fast path of the quantize kernels in each mode, on data
    # crowded around rounding ties, against the oracle in the same mode.
    import numpy as np
    rng = np.random.default_rng(40 + flags)
    x = rng.normal(0, 2, size=(257, 1031)).astype(np.float32)
    L = gpu.lib()
    L.omcudaSetQuantizationMode(flags)
    orc.L.orc_set_quant_mode(flags)
    try:
        yq, s, z = gpu.dynamic_quantize_linear(x)
        wq, ws, wz = orc.dynamic_quantize_linear(x)
        assert s.tobytes() == ws.tobytes() and int(z) == int(wz)
        assert np.array_equal(yq, wq)
        # QuantizeLinear with a scale whose reciprocal is inexact, ties included
        scale = np.float32(0.0123)
        t = ((rng.integers(-300, 300, x.size) + 0.5) * scale).astype(np.float32).reshape(x.shape)
        t += (rng.integers(-2, 3, x.shape) * np.spacing(t)).astype(np.float32)
        for dt, zp in ((np.uint8, 131), (np.int8, -7)):
            got = gpu.quantize_linear(t, scale, np.array(zp, dt), out_dtype=dt)
            want = orc.quantize(t, scale, zp, signed=(dt == np.int8))
            assert np.array_equal(got, want), (dt, int((got != want).sum()))
        d = gpu.dequantize_linear(wq, ws, np.array(9, np.uint8))
        assert d.tobytes() == orc.dequantize_linear(wq, ws, 9).tobytes()
    finally:
        L.omcudaSetQuantizationMode(0)
        orc.L.orc_set_quant_mode(0)

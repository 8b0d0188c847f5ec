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

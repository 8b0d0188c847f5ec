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

"""The CPU oracle against the known-answer vectors onnx-mlir's own lit tests
hold (tests/golden/lit_kats.json, extracted by tests/golden/make_lit_kats.py)
and against properties of the lowering it restates."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
KATS = json.load(open(os.path.join(HERE, "golden", "lit_kats.json")))["cases"]
NP = {"ui8": np.uint8, "i8": np.int8, "i32": np.int32, "f32": np.float32}


def arr(t):
    if t is None:
        return None
    return np.array(t["data"], dtype=NP[t["dtype"]]).reshape(t["shape"])


@pytest.mark.parametrize("kat", [k for k in KATS if k["op"] == "MatMulInteger"],
                         ids=lambda k: k["name"])
def test_matmulinteger_lit_vectors(orc, kat):
    A, B = arr(kat["A"]), arr(kat["B"])
    got = orc.matmul_integer(A, B, arr(kat["a_zero_point"]),
                             arr(kat["b_zero_point"]))
    want = arr(kat["expected"])
    assert got.shape == want.shape
    assert np.array_equal(got, want)


def test_round_lit_vector(orc):
    kat = [k for k in KATS if k["op"] == "Round"][0]
    x = arr(kat["X"])
    got = np.array([orc.round_even(v) for v in x], np.float32)
    assert np.array_equal(got, arr(kat["expected"]))


def test_round_even_equals_rint_for_every_float(orc):
    # Justifies using the hardware round-to-nearest-even on the GPU in place of
    # the reference's floor-based emulation.
    assert orc.L.orc_selftest_round_even_exhaustive() == 0


def test_round_even_ties(orc):
    for x, want in [(0.5, 0.0), (1.5, 2.0), (2.5, 2.0), (-0.5, 0.0), (-1.5, -2.0),
                    (-2.5, -2.0), (254.5, 254.0), (255.5, 256.0), (1e10, 1e10)]:
        assert orc.round_even(x) == np.float32(want)


def test_dql_matches_onnx_formula(orc):
    # ONNX operator definition: scale = (max(0,max) - min(0,min)) / 255,
    # zp = clip(round(0 - min/scale)), y = clip(round(x/scale) + zp).
    rng = np.random.default_rng(0)
    for _ in range(20):
        x = rng.normal(0, rng.uniform(0.1, 5), size=rng.integers(1, 300)).astype(np.float32)
        y, s, z = orc.dynamic_quantize_linear(x)
        mx, mn = max(x.max(), np.float32(0)), min(x.min(), np.float32(0))
        s_want = np.float32(np.float32(mx - mn) / np.float32(255))
        assert s == s_want
        z_want = np.clip(np.rint(np.float32(0) - np.float32(mn / s_want)), 0, 255)
        assert int(z) == int(z_want)
        y_want = np.clip(np.rint((x / s_want).astype(np.float32)) + np.float32(z_want), 0, 255)
        assert np.array_equal(y, y_want.astype(np.uint8))


def test_dql_edge_cases(orc):
    # all zeros: scale 0, 0/0 = NaN everywhere, clip turns NaN into 0
    y, s, z = orc.dynamic_quantize_linear(np.zeros(17, np.float32))
    assert s == 0 and z == 0 and not y.any()
    # all positive: range extended to include 0, zero point 0
    y, s, z = orc.dynamic_quantize_linear(np.array([1, 2, 3], np.float32))
    assert z == 0 and s == np.float32(3) / np.float32(255) and y[-1] == 255
    # all negative: zero point 255
    y, s, z = orc.dynamic_quantize_linear(np.array([-1, -2, -4], np.float32))
    assert z == 255 and y.min() == 0
    # NaN is ignored by the min/max reduction and quantizes to 0
    y, s, z = orc.dynamic_quantize_linear(np.array([np.nan, -1, 1], np.float32))
    assert s == np.float32(2) / np.float32(255) and y[0] == 0
    # single element / rank 0
    y, s, z = orc.dynamic_quantize_linear(np.array(2.0, np.float32))
    assert y.shape == () and y == 255


def test_matmul_integer_zero_point_forms(orc):
    rng = np.random.default_rng(1)
    A = rng.integers(0, 256, (7, 19), dtype=np.uint8)
    B = rng.integers(-128, 128, (19, 5), dtype=np.int8)
    az_row = rng.integers(0, 256, 7, dtype=np.uint8)
    bz_col = rng.integers(-128, 128, 5, dtype=np.int8)
    want = (A.astype(np.int64) - az_row[:, None]) @ (B.astype(np.int64) - bz_col[None, :])
    got = orc.matmul_integer_2d(A, B, az_row, bz_col)
    assert np.array_equal(got, want.astype(np.int32))
    got = orc.matmul_integer_2d(A, B, np.array([3], np.uint8), None)
    assert np.array_equal(got, ((A.astype(np.int64) - 3) @ B.astype(np.int64)).astype(np.int32))


def test_qlinear_matmul_wraps_instead_of_saturating(orc):
    # The reference truncates the i32 result to 8 bits (QLinearMatMul.cpp:131-138).
    A = np.full((1, 4), 255, np.uint8)
    B = np.full((4, 1), 127, np.int8)
    y = orc.qlinear_matmul(A, 1.0, np.uint8(0), B, np.array([1.0], np.float32),
                           np.zeros(1, np.int8), 1.0, np.uint8(0))
    acc = 4 * 255 * 127
    assert y.dtype == np.uint8 and int(y[0, 0]) == acc % 256
    y = orc.qlinear_matmul(A.astype(np.int8) // 2, 1.0, np.int8(0), B,
                           np.array([1.0], np.float32), np.zeros(1, np.int8), 1.0,
                           np.int8(5))
    a8 = (A.astype(np.int8) // 2).astype(np.int64)
    acc = int((a8 @ B.astype(np.int64))[0, 0]) + 5
    assert y.dtype == np.int8 and int(y[0, 0]) == ((acc + 128) % 256) - 128


def test_qlinear_matmul_in_range_matches_spec(orc):
    rng = np.random.default_rng(2)
    A = rng.integers(0, 256, (6, 32), dtype=np.uint8)
    B = rng.integers(-127, 128, (32, 9), dtype=np.int8)
    bs = rng.uniform(1e-3, 2e-3, 9).astype(np.float32)
    y = orc.qlinear_matmul(A, 0.02, np.uint8(128), B, bs, np.zeros(9, np.int8), 0.5,
                           np.uint8(128))
    acc = (A.astype(np.int64) - 128) @ B.astype(np.int64)
    S = ((np.float32(0.02) * bs) / np.float32(0.5)).astype(np.float32)
    want = np.rint(acc.astype(np.float32) * S[None, :]).astype(np.int64) + 128
    assert want.min() >= 0 and want.max() <= 255
    assert np.array_equal(y, want.astype(np.uint8))


def test_reference_shaped_baseline_agrees(orc):
    rng = np.random.default_rng(3)
    A = rng.integers(0, 256, (13, 37), dtype=np.uint8)
    B = rng.integers(-127, 128, (37, 21), dtype=np.int8)
    want = orc.matmul_integer_2d(A, B, np.array([77], np.uint8), None)
    assert np.array_equal(orc.ref_shaped_matmul_integer(A, B, 77, threads=1), want)
    assert np.array_equal(orc.ref_shaped_matmul_integer(A, B, 77, threads=4), want)


def test_fp32_ops_against_numpy(orc):
    rng = np.random.default_rng(4)
    x = rng.normal(size=(5, 33)).astype(np.float32)
    e = np.exp(x - x.max(-1, keepdims=True))
    assert np.allclose(orc.softmax(x), e / e.sum(-1, keepdims=True), rtol=1e-5)
    g, b = rng.normal(size=33).astype(np.float32), rng.normal(size=33).astype(np.float32)
    ln = (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5) * g + b
    assert np.allclose(orc.layernorm(x, g, b), ln, rtol=1e-4, atol=1e-5)
    from math import erf
    ge = np.array([0.5 * v * (1 + erf(v / np.sqrt(2))) for v in x.ravel()]).reshape(x.shape)
    assert np.allclose(orc.gelu(x), ge, rtol=1e-5, atol=1e-6)
    t = rng.normal(size=(2, 3, 4, 5)).astype(np.float32)
    assert np.array_equal(orc.transpose_0213(t), t.transpose(0, 2, 1, 3))
    a, bm = rng.normal(size=(3, 4, 6)).astype(np.float32), rng.normal(size=(3, 6, 5)).astype(np.float32)
    assert np.allclose(orc.matmul_f32(a, bm), a @ bm, rtol=1e-5, atol=1e-5)
    q, k, v = (rng.normal(size=(2, 7, 8)).astype(np.float32) for _ in range(3))
    out = orc.attention(q, k, v, 2, 0.5)
    qh, kh, vh = (z.reshape(2, 7, 2, 4).transpose(0, 2, 1, 3) for z in (q, k, v))
    sc = qh @ kh.transpose(0, 1, 3, 2) * 0.5
    p = np.exp(sc - sc.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    want = (p @ vh).transpose(0, 2, 1, 3).reshape(2, 7, 8)
    assert np.allclose(out, want, rtol=1e-5, atol=1e-6)


# ---- vectors from executing the reference's expected Krnl IR ------------------------

import lit_ir_cases  # noqa: E402


@pytest.mark.parametrize("case", lit_ir_cases.CASES, ids=lit_ir_cases.case_id)
def test_oracle_matches_executed_lit_ir(orc, case):
    got, want = lit_ir_cases.run_case(case, lit_ir_cases.OracleBackend(orc))
    lit_ir_cases.assert_same(got, want)


@pytest.mark.parametrize("case", lit_ir_cases.FP32_CASES, ids=lit_ir_cases.fp32_case_id)
def test_oracle_fp32_ops_match_executed_lit_ir(orc, case):
    # Softmax, MatMul and Gelu: the oracle performs the reference's fp32
    # operations in the reference's order (and calls the same libm), so it
    # must reproduce the executed IR bit for bit.  LayerNormalization: the
    # reference's SIMD lowering sums in vector lanes, the oracle in order, so
    # only the last bits of the two reductions differ.
    got, want, kind, _ = lit_ir_cases.run_fp32_case(case, lit_ir_cases.OracleFp32Backend(orc))
    assert got.shape == want.shape
    if kind == "layernorm":
        assert np.allclose(got, want, rtol=1e-5, atol=1e-5), np.abs(got - want).max()
    else:
        assert got.tobytes() == want.tobytes(), np.abs(got - want).max()


@pytest.mark.parametrize("case", lit_ir_cases.MODE_CASES, ids=lit_ir_cases.mode_case_id)
def test_oracle_modes_match_executed_lit_ir(orc, case):
    # --disable-quantization-zero-point and enable-fast-math, against the
    # executed IR of the reference's lowering tests for those options.
    orc.L.orc_set_quant_mode(lit_ir_cases.MODE_FLAGS[case["mode"]])
    try:
        got, want = lit_ir_cases.run_case(case, lit_ir_cases.OracleBackend(orc))
    finally:
        orc.L.orc_set_quant_mode(0)
    lit_ir_cases.assert_same(got, want)
    if case["mode"] == "fast_math":
        # the fixture tells the modes apart: the default arithmetic must not match
        got0, _ = lit_ir_cases.run_case(case, lit_ir_cases.OracleBackend(orc))
        assert got0[0].tobytes() != want[0].tobytes()

"""GPU parity: MatMulInteger, QLinearMatMul and the fused dynamic-quantized
linear through the C ABI against the CPU oracle.  Bit-exact for int32 / uint8
results; fp32 dequantized outputs are expected bit-exact too and are checked
at the 1e-5 relative tolerance the path's contract states."""
import json
import os

import numpy as np
import pytest

from gpu_util import DevGemm

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
KATS = json.load(open(os.path.join(HERE, "golden", "lit_kats.json")))["cases"]
NP = {"ui8": np.uint8, "i8": np.int8, "i32": np.int32, "f32": np.float32}


def arr(t):
    return None if t is None else np.array(t["data"], dtype=NP[t["dtype"]]).reshape(t["shape"])


def rand8(rng, shape, dt):
    if dt == np.uint8:
        return rng.integers(0, 256, shape, dtype=np.uint8)
    return rng.integers(-128, 128, shape, dtype=np.int8)


@pytest.mark.parametrize("kat", [k for k in KATS if k["op"] == "MatMulInteger"],
                         ids=lambda k: k["name"])
def test_lit_vectors(gpu, kat):
    A, B = arr(kat["A"]), arr(kat["B"])
    want = arr(kat["expected"])
    got = gpu.matmul_integer(A, B, arr(kat["a_zero_point"]), arr(kat["b_zero_point"]))
    assert np.array_equal(got.reshape(want.shape), want)


SHAPES = [(1, 16, 8), (1, 768, 768), (16, 4096, 512), (5, 7, 3), (127, 100, 33),
          (128, 128, 256), (129, 144, 264), (300, 768, 100), (256, 1024, 640),
          (513, 48, 1000), (128, 768, 768)]


@pytest.mark.parametrize("choice", [1, 2], ids=["tcgen05", "simt"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_matmul_integer_kernels(gpu, orc, shape, choice):
    M, K, N = shape
    if choice == 1 and K % 16:
        pytest.skip("tensor-core kernel needs K % 16 == 0; the SIMT kernel covers it")
    rng = np.random.default_rng(M * 31 + K * 7 + N)
    A, B = rand8(rng, (M, K), np.uint8), rand8(rng, (K, N), np.int8)
    az = rng.integers(0, 256, 1, dtype=np.uint8)
    dg = DevGemm(gpu)
    want = orc.matmul_integer_2d(A, B, az, None)
    got = dg.matmul_integer(A, B, az, None, choice)
    assert np.array_equal(got, want), np.argwhere(got != want)[:8]


@pytest.mark.parametrize("choice", [1, 2], ids=["tcgen05", "simt"])
@pytest.mark.parametrize("adt,bdt", [(np.uint8, np.uint8), (np.int8, np.int8),
                                     (np.int8, np.uint8), (np.uint8, np.int8)])
def test_signedness_and_zero_point_forms(gpu, orc, adt, bdt, choice):
    rng = np.random.default_rng(11)
    M, K, N = 130, 160, 72
    A, B = rand8(rng, (M, K), adt), rand8(rng, (K, N), bdt)
    dg = DevGemm(gpu)
    for az, bz in [(None, None), (rand8(rng, 1, adt), None), (None, rand8(rng, 1, bdt)),
                   (rand8(rng, M, adt), rand8(rng, N, bdt)),
                   (rand8(rng, 1, adt), rand8(rng, N, bdt))]:
        want = orc.matmul_integer_2d(A, B, az, bz)
        got = dg.matmul_integer(A, B, az, bz, choice)
        assert np.array_equal(got, want)


@pytest.mark.parametrize("choice", [0, 2], ids=["auto", "simt"])
@pytest.mark.parametrize("adt,bdt", [(np.uint8, np.uint8), (np.int8, np.int8),
                                     (np.int8, np.uint8), (np.uint8, np.int8)])
def test_gemv_shaped_rows_1_to_32(gpu, orc, adt, bdt, choice):
    # The GEMV-shaped kernels (dp4a for one row, mma.sync m16n8k32 with a
    # permuted K order for 2..16) and the hand-over to the tensor-core kernels
    # above 16 rows: ragged M, K (not a multiple of 16 / of the 64-byte block /
    # of a warp's run of blocks) and N (not a multiple of the 16 columns of a
    # block, more blocks than SMs), every signedness and zero-point form.
    rng = np.random.default_rng(41)
    dg = DevGemm(gpu)
    for M, K, N in [(1, 100, 33), (3, 1040, 17), (5, 7, 3), (8, 64, 16), (9, 144, 40),
                    (13, 2000, 70), (16, 4160, 136), (16, 2048, 1000), (2, 16, 8),
                    (7, 1024, 2400), (16, 13312, 48), (23, 1168, 72), (32, 3072, 520)]:
        A, B = rand8(rng, (M, K), adt), rand8(rng, (K, N), bdt)
        for az, bz in [(None, None), (rand8(rng, 1, adt), None),
                       (rand8(rng, M, adt), rand8(rng, N, bdt))]:
            want = orc.matmul_integer_2d(A, B, az, bz)
            got = dg.matmul_integer(A, B, az, bz, choice)
            assert np.array_equal(got, want), (M, K, N, np.argwhere(got != want)[:8])


@pytest.mark.parametrize("M,K,N", [(17, 8192, 256), (100, 8208, 260), (128, 16384, 512),
                                   (129, 8192, 512), (300, 8208, 768), (512, 9216, 1024)])
def test_split_k_shapes(gpu, orc, M, K, N):
    # Up to 512 rows, with few output tiles and K of 8192 or more, the
    # tensor-core kernels deal each tile's K loop to several work units (raw partial sums through a
    # workspace, then one reduce pass with the real tail): on single CTAs up to
    # 128 rows, on CTA pairs above.  All three tails against the oracle, every
    # zero-point form, K not a multiple of the 128-byte K step.
    rng = np.random.default_rng(M + K + N)
    dg = DevGemm(gpu)
    for adt, bdt in [(np.uint8, np.int8), (np.int8, np.uint8)]:
        A, B = rand8(rng, (M, K), adt), rand8(rng, (K, N), bdt)
        for az, bz in [(None, None), (rand8(rng, 1, adt), None),
                       (rand8(rng, M, adt), rand8(rng, N, bdt))]:
            want = orc.matmul_integer_2d(A, B, az, bz)
            for choice in (0, 1):
                got = dg.matmul_integer(A, B, az, bz, choice)
                assert np.array_equal(got, want), (adt, choice, np.argwhere(got != want)[:8])
    # DEQUANT tail (DynamicQuantizeLinear -> MatMulInteger -> Cast -> Mul -> Add)
    X = rng.normal(size=(M, K)).astype(np.float32)
    W = rng.integers(-127, 128, (K, N), dtype=np.int8)
    bias = rng.normal(0, 0.02, N).astype(np.float32)
    ref = orc.dyn_quant_linear(X, W, np.float32(0.0157), bias)
    Y = gpu.dyn_quant_linear(X, W, np.float32(0.0157), None, bias, 0)
    assert Y.tobytes() == ref["Y"].tobytes()
    # REQUANT tail (QLinearMatMul), per-column scales and zero points
    A, B, bs, bz = qlinear_case(rng, (M,), K, N)
    args = (A, np.float32(0.02), np.uint8(128), B, bs, bz, np.float32(0.5), np.uint8(128))
    assert np.array_equal(gpu.qlinear_matmul(*args), orc.qlinear_matmul(*args))


def test_matmul_integer_api_shapes(gpu, orc):
    rng = np.random.default_rng(12)
    # 3-D A times 2-D B (the encoder's broadcast-A form), host and device tensors
    A, B = rand8(rng, (4, 33, 64), np.uint8), rand8(rng, (64, 48), np.int8)
    az = np.array(7, np.uint8)
    want = orc.matmul_integer(A, B, az, None)
    assert np.array_equal(gpu.matmul_integer(A, B, az, None), want)
    assert np.array_equal(gpu.matmul_integer(A, B, az, None, device=True).numpy(), want)
    # equal batch dims on both sides
    A, B = rand8(rng, (3, 17, 32), np.int8), rand8(rng, (3, 32, 20), np.int8)
    assert np.array_equal(gpu.matmul_integer(A, B), orc.matmul_integer(A, B))
    # vector operands
    a, b = rand8(rng, 32, np.uint8), rand8(rng, (32, 9), np.int8)
    assert np.array_equal(gpu.matmul_integer(a, b), orc.matmul_integer(a, b))
    # numpy broadcasting of the batch dimensions (ONNXOps/Math/MatMul.cpp:46-166):
    # size-1 and missing dimensions on either side, a vector against a batch
    for sa, sb in (((4, 1, 5, 16), (3, 16, 7)), ((3, 5, 16), (2, 1, 16, 7)),
                   ((16,), (2, 3, 16, 7)), ((2, 3, 5, 16), (16,)),
                   ((1, 5, 16), (6, 16, 7)), ((2, 3, 5, 16), (2, 3, 16, 7))):
        A, B = rand8(rng, sa, np.uint8), rand8(rng, sb, np.int8)
        az, bz = np.array(9, np.uint8), np.array(-3, np.int8)
        want = orc.matmul_integer(A, B, az, bz)
        got = gpu.matmul_integer(A, B, az, bz)
        assert got.shape == want.shape and np.array_equal(got, want), (sa, sb)
        assert np.array_equal(gpu.matmul_integer(A, B, az, bz, device=True).numpy(), want)
    with pytest.raises(gpu.OmcudaError) as ei:
        gpu.matmul_integer(rand8(rng, (2, 5, 16), np.uint8), rand8(rng, (3, 16, 7), np.int8))
    assert ei.value.code == gpu.EINVAL
    # per-row a zero point, per-column b zero point
    A, B = rand8(rng, (21, 32), np.uint8), rand8(rng, (32, 9), np.uint8)
    az, bz = rand8(rng, 21, np.uint8), rand8(rng, 9, np.uint8)
    assert np.array_equal(gpu.matmul_integer(A, B, az, bz), orc.matmul_integer_2d(A, B, az, bz))


def test_worst_case_magnitude_k14336(gpu, orc):
    # |acc| <= 255 * 128 * 14336 < 2^31: no overflow at the largest K of the sweep
    M, K, N = 64, 14336, 128
    A = np.full((M, K), 255, np.uint8)
    B = np.full((K, N), -128, np.int8)
    B[:, ::2] = 127
    dg = DevGemm(gpu)
    want = orc.matmul_integer_2d(A, B, None, None)
    assert np.array_equal(dg.matmul_integer(A, B, None, None, 1), want)
    assert np.array_equal(dg.matmul_integer(A, B, None, None, 2), want)


def test_full_size_4096_checksums(gpu):
    # Size-independent property at the headline GEMM size: row and column sums
    # of Y equal A @ rowsum(B) and colsum(A) @ B, computed exactly in int64.
    rng = np.random.default_rng(13)
    M = N = K = 4096
    A = rng.integers(0, 256, (M, K), dtype=np.uint8)
    B = rng.integers(-127, 128, (K, N), dtype=np.int8)
    az = np.array([113], np.uint8)
    Y = DevGemm(gpu).matmul_integer(A, B, az, None, 1).astype(np.int64)
    As = A.astype(np.int64) - 113
    assert np.array_equal(Y.sum(1), As @ B.astype(np.int64).sum(1))
    assert np.array_equal(Y.sum(0), As.sum(0) @ B.astype(np.int64))


def qlinear_case(rng, lead, K, N, per_column=True):
    A = rng.integers(0, 256, lead + (K,), dtype=np.uint8)
    B = rng.integers(-127, 128, (K, N), dtype=np.int8)
    bs = rng.uniform(0.001, 0.01, N if per_column else 1).astype(np.float32)
    bz = np.zeros(N if per_column else 1, np.int8)
    return A, B, bs, bz


def test_qlinear_matmul_small_with_wrap(gpu, orc):
    rng = np.random.default_rng(14)
    A, B, bs, bz = qlinear_case(rng, (3, 50), 256, 96)
    bs = (bs * np.float32(16)).astype(np.float32)  # widen so results leave [0,255]
    args = (A, np.float32(0.02), np.uint8(128), B, bs, bz, np.float32(0.5), np.uint8(128))
    want = orc.qlinear_matmul(*args)
    # make sure the case reaches outside [0,255] before the truncation
    acc = (A.reshape(-1, 256).astype(np.int64) - 128) @ B.astype(np.int64)
    pre = np.rint(acc * ((np.float32(0.02) * bs) / np.float32(0.5))[None, :]) + 128
    assert (pre > 255).any() and (pre < 0).any()
    got = gpu.qlinear_matmul(*args)
    assert np.array_equal(got, want)
    bz2 = rng.integers(-5, 6, 96, dtype=np.int8)
    args2 = (A, np.float32(0.02), np.uint8(120), B, bs, bz2, np.float32(0.5), np.uint8(3))
    assert np.array_equal(gpu.qlinear_matmul(*args2), orc.qlinear_matmul(*args2))


def test_qlinear_matmul_int8_output_scalar_scale(gpu, orc):
    rng = np.random.default_rng(15)
    A = rng.integers(-128, 128, (40, 64), dtype=np.int8)
    B = rng.integers(-128, 128, (64, 24), dtype=np.int8)
    args = (A, np.float32(0.1), np.int8(-4), B, np.array([0.05], np.float32),
            np.array([2], np.int8), np.float32(0.7), np.int8(-9))
    assert np.array_equal(gpu.qlinear_matmul(*args), orc.qlinear_matmul(*args))


def test_config2_qlinear_matmul_full_size(gpu, orc):
    # A u8 [32,512,1024], B i8 [1024,4096], per-column b_scale: the whole
    # output on the GPU, a seeded sample of 192 rows against the oracle, plus a
    # byte histogram sanity check that the wrap region is populated.
    rng = np.random.default_rng(42)
    A, B, bs, bz = qlinear_case(rng, (32, 512), 1024, 4096)
    args = (np.float32(0.02), np.uint8(128), B, bs, bz, np.float32(0.5), np.uint8(128))
    got = gpu.qlinear_matmul(A, *args).reshape(-1, 4096)
    rows = rng.choice(32 * 512, 192, replace=False)
    want = orc.qlinear_matmul(A.reshape(-1, 1024)[rows], *args)
    assert np.array_equal(got[rows], want)


def test_config1_dyn_quant_linear(gpu, orc):
    rng = np.random.default_rng(42)
    X = rng.normal(size=(128, 768)).astype(np.float32)
    W = rng.integers(-127, 128, (768, 768), dtype=np.int8)
    bias = rng.normal(0, 0.02, 768).astype(np.float32)
    w_scale = np.float32(0.0157)
    ref = orc.dyn_quant_linear(X, W, w_scale, bias)
    # step by step, as the unfused graph runs
    xq, xs, xz = gpu.dynamic_quantize_linear(X)
    assert np.array_equal(xq, ref["xq"]) and xs == ref["x_scale"] and xz == ref["x_zp"]
    acc = gpu.matmul_integer(xq, W, xz, None)
    assert np.array_equal(acc, ref["acc"])
    # fused
    Y = gpu.dyn_quant_linear(X, W, w_scale, None, bias, 0)
    assert np.allclose(Y, ref["Y"], rtol=1e-5, atol=0)
    assert Y.tobytes() == ref["Y"].tobytes()
    Yd = gpu.dyn_quant_linear(X, W, w_scale, None, bias, 0, device=True).numpy()
    assert Yd.tobytes() == ref["Y"].tobytes()


def test_dyn_quant_linear_forms(gpu, orc):
    rng = np.random.default_rng(16)
    X = rng.normal(size=(2, 37, 96)).astype(np.float32)
    W = rng.integers(-127, 128, (96, 40), dtype=np.int8)
    ref = orc.dyn_quant_linear(X, W, 0.01, None)
    # form 1: (acc * x_scale) * w_scale, two roundings on the tensor
    want1 = orc.dequant_tail(ref["acc"], ref["x_scale"], np.float32(0.01), 1, None)
    got1 = gpu.dyn_quant_linear(X, W, np.float32(0.01), None, None, 1)
    assert got1.tobytes() == want1.tobytes()
    # per-column weight scale
    ws = rng.uniform(0.005, 0.02, 40).astype(np.float32)
    s = (ref["x_scale"] * ws).astype(np.float32)
    want = (ref["acc"].astype(np.float32) * s).astype(np.float32)
    got = gpu.dyn_quant_linear(X, W, ws, None, None, 0)
    assert got.tobytes() == want.tobytes()
    # weight zero point
    wz = np.array(3, np.int8)
    acc = orc.matmul_integer(ref["xq"], W, ref["x_zp"], wz)
    want = orc.dequant_tail(acc, ref["x_scale"] * np.float32(0.01), 0.0, 0, None)
    got = gpu.dyn_quant_linear(X, W, np.float32(0.01), wz, None, 0)
    assert got.tobytes() == want.tobytes()


@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 14336), (14336, 4096)])
@pytest.mark.parametrize("M", [1, 16, 256, 4096, 16384])
def test_config3_sweep_members(gpu, orc, M, K, N):
    # Every member of the MatMulInteger sweep: DynamicQuantizeLinear over the
    # whole X, then sampled rows of the GEMM and of the dequantized output
    # against the oracle.
    rng = np.random.default_rng(M + K + N)
    X = rng.standard_normal((M, K), dtype=np.float32)
    W = rng.integers(-127, 128, (K, N), dtype=np.int8)
    w_scale = np.float32(0.02 * 4 / 127)
    xq, xs, xz = orc.dynamic_quantize_linear(X)
    Y = gpu.dyn_quant_linear(X, W, w_scale, None, None, 0)
    rows = rng.choice(M, min(M, 48), replace=False)
    acc = orc.matmul_integer_2d(xq[rows], W, xz.reshape(1), None)
    want = orc.dequant_tail(acc, xs * w_scale, 0.0, 0, None)
    assert np.allclose(Y[rows], want, rtol=1e-5, atol=0)
    assert Y[rows].tobytes() == want.tobytes()


def bf16_split(x):
    """hi = bf16(x), lo = bf16(x - hi), round to nearest even, as uint16 bit
    patterns (numpy has no bfloat16)."""
    def to_bf16_bits(f):
        u = f.astype(np.float32).view(np.uint32).astype(np.uint64)
        r = (u + 0x7fff + ((u >> 16) & 1)) >> 16
        return r.astype(np.uint16)
    hi = to_bf16_bits(x)
    hi_f = (hi.astype(np.uint32) << 16).view(np.float32)
    lo = to_bf16_bits((x - hi_f).astype(np.float32))
    return hi, lo


@pytest.mark.parametrize("M,K,N", [(300, 256, 192), (512, 1024, 3072), (33, 64, 72)])
def test_dequant_split_epilogue_equals_split_of_dequant(gpu, M, K, N):
    # The tail that writes bf16 hi/lo planes (operands of the tensor-core
    # attention kernel) must hold exactly the split of the f32 dequant tail.
    from gpu_util import DevGemm
    rng = np.random.default_rng(M + N)
    dg = DevGemm(gpu)
    A = rng.integers(0, 256, (M, K), dtype=np.uint8)
    B = rng.integers(-127, 128, (K, N), dtype=np.int8)
    pb, keep = dg.prepare(B)
    dA = dg.dtensor(A)
    az = dg.dtensor(np.array([131], np.uint8))
    sa = dg.dtensor(np.array([0.013], np.float32))
    sb = dg.dtensor(rng.uniform(0.001, 0.01, N).astype(np.float32))
    bias = dg.dtensor(rng.normal(0, 0.5, N).astype(np.float32))
    g = dg.dev.GemmArgs()
    g.M, g.N, g.K = M, N, K
    g.A, g.a_signed, g.B = dA.data_ptr, 0, pb
    g.a_zp, g.a_zp_len = az.data_ptr, 1
    g.sa, g.sb, g.sb_len, g.bias = sa.data_ptr, sb.data_ptr, N, bias.data_ptr
    g.kernel_choice = dg.dev.KERNEL_TENSOR_CORE
    Y = gpu.Tensor.device_empty((M, N), np.float32)
    g.epilogue, g.Y = dg.dev.EPI_DEQUANT, Y.data_ptr
    dg.dev.gemm_i8(g, dg.stream)
    P = gpu.Tensor.device_empty((2, M, N), np.uint16)
    g.epilogue, g.Y = dg.dev.EPI_DEQUANT_SPLIT, P.data_ptr
    dg.dev.gemm_i8(g, dg.stream)
    y, planes = Y.numpy(), P.numpy()
    gpu.synchronize()
    hi, lo = bf16_split(y)
    assert np.array_equal(planes[0], hi)
    assert np.array_equal(planes[1], lo)
    # and the standalone split kernel writes the same planes
    P2 = gpu.Tensor.device_empty((2, M, N), np.uint16)
    if N % 4 == 0:
        dg.dev.split_bf16(Y.data_ptr, M, N, N, P2.data_ptr, P2.data_ptr + 2 * M * N,
                          N, 0, dg.stream)
        assert np.array_equal(P2.numpy(), planes)


@pytest.mark.parametrize("M,K,N,gelu", [(300, 256, 192, 1), (1024, 1024, 4096, 1),
                                        (33, 64, 72, 0), (515, 512, 1000, 1),
                                        (2600, 512, 1800, 1)])
def test_range_then_quantizing_tails_equal_dequant_then_quantize(gpu, M, K, N, gelu):
    # "linear -> DynamicQuantizeLinear" run as two passes over the product
    # (range only, then quantize while storing uint8) must give the bytes,
    # scale and zero point of the f32 tail followed by the quantize kernel.
    from gpu_util import DevGemm
    rng = np.random.default_rng(M * 7 + N)
    dg = DevGemm(gpu)
    A = rng.integers(0, 256, (M, K), dtype=np.uint8)
    B = rng.integers(-127, 128, (K, N), dtype=np.int8)
    pb, keep = dg.prepare(B)
    dA = dg.dtensor(A)
    az = dg.dtensor(np.array([128], np.uint8))
    sa = dg.dtensor(np.array([0.011], np.float32))
    sb = dg.dtensor(np.array([0.0004], np.float32))
    bias = dg.dtensor(rng.normal(0, 0.5, N).astype(np.float32))
    g = dg.dev.GemmArgs()
    g.M, g.N, g.K = M, N, K
    g.A, g.a_signed, g.B = dA.data_ptr, 0, pb
    g.a_zp, g.a_zp_len = az.data_ptr, 1
    g.sa, g.sb, g.sb_len, g.bias, g.gelu = sa.data_ptr, sb.data_ptr, 1, bias.data_ptr, gelu
    g.kernel_choice = dg.dev.KERNEL_TENSOR_CORE
    ranges = gpu.Tensor.device_empty((4,), np.int32)
    dg.dev.range_init(ranges.data_ptr, 2, dg.stream)
    # reference chain: f32 tail with running range, then the quantize kernel
    Y = gpu.Tensor.device_empty((M, N), np.float32)
    g.epilogue, g.Y, g.out_minmax = dg.dev.EPI_DEQUANT, Y.data_ptr, ranges.data_ptr
    dg.dev.gemm_i8(g, dg.stream)
    q_ref = gpu.Tensor.device_empty((M, N), np.uint8)
    par_ref = gpu.Tensor.device_empty((4,), np.float32)
    dg.dev.quantize_from_range(Y.data_ptr, M * N, ranges.data_ptr, q_ref.data_ptr,
                               par_ref.data_ptr, par_ref.data_ptr + 8,
                               par_ref.data_ptr + 12, dg.stream)
    # two passes over the product, no f32 tensor
    g.epilogue, g.Y, g.out_minmax = dg.dev.EPI_DEQUANT_RANGE, None, ranges.data_ptr + 8
    dg.dev.gemm_i8(g, dg.stream)
    q = gpu.Tensor.device_empty((M, N), np.uint8)
    par = gpu.Tensor.device_empty((4,), np.float32)
    g.epilogue, g.Y, g.out_minmax = dg.dev.EPI_DEQUANT_QUANT, q.data_ptr, None
    g.q_range, g.q_params = ranges.data_ptr + 8, par.data_ptr
    g.q_scale, g.q_zp = par.data_ptr + 8, par.data_ptr + 12
    dg.dev.gemm_i8(g, dg.stream)
    r = ranges.numpy()
    gpu.synchronize()
    assert r[0] == r[2] and r[1] == r[3]
    # slots: scale, zero point as float, y_scale, first byte = y_zero_point
    pw, pw_ref = par.numpy().view(np.uint32), par_ref.numpy().view(np.uint32)
    assert np.array_equal(pw[:3], pw_ref[:3]) and (pw[3] & 0xff) == (pw_ref[3] & 0xff)
    assert np.array_equal(q.numpy(), q_ref.numpy())
    # and the bytes are DynamicQuantizeLinear of the f32 tensor (numpy restatement)
    y = Y.numpy()
    scale = np.float32(np.float32(max(y.max(), 0) - min(y.min(), 0)) / np.float32(255))
    assert par.numpy()[0] == scale


@pytest.mark.parametrize("M,K,N", [(4096, 4096, 4096), (5000, 2048, 4104), (300, 512, 1000),
                                   (2600, 512, 1800), (9300, 256, 2048)])
def test_whole_output_checksums(gpu, orc, M, K, N):
    # Every tile of the output is stored exactly once (the epilogue leaves
    # through TMA stores that clip ragged edges): sampled rows against the
    # oracle and column sums of the whole result against exact integer sums.
    # 4096^3, 2600 x 1800 and 9300 x 2048 end in a round of 256 x 128 half
    # tiles on the 2-CTA kernel (the last two with ragged edges).
    from gpu_util import DevGemm
    rng = np.random.default_rng(K + N)
    A = rng.integers(0, 256, (M, K), dtype=np.uint8)
    B = rng.integers(-127, 128, (K, N), dtype=np.int8)
    dg = DevGemm(gpu)
    rows = np.concatenate([np.arange(0, 40), np.arange(max(M - 300, 40), M, 7)])
    want = orc.matmul_integer_2d(A[rows], B, np.array([117], np.uint8), None)
    Y = dg.matmul_integer(A, B, 117, None, 1)
    assert np.array_equal(Y[rows], want)
    As = A.astype(np.int64) - 117
    assert np.array_equal(Y.astype(np.int64).sum(0), As.sum(0) @ B.astype(np.int64))

@pytest.mark.parametrize("M,K,N,choice", [(300, 256, 192, 1), (260, 512, 1000, 1), (3, 100, 70, 2),
                                          (13, 200, 70, 2), (16, 1040, 136, 0)])
def test_dequant_tail_with_residual(gpu, M, K, N, choice):
    # y = tail(acc) + residual, the onnx.Add of a residual connection folded
    # into the GEMM: one more separately rounded fp32 add, so it must equal
    # the sum of the plain tail's result and the residual bit for bit.
    from gpu_util import DevGemm
    rng = np.random.default_rng(M * N)
    dg = DevGemm(gpu)
    A = rng.integers(0, 256, (M, K), dtype=np.uint8)
    B = rng.integers(-127, 128, (K, N), dtype=np.int8)
    res = rng.normal(0, 1, (M, N)).astype(np.float32)
    pb, keep = dg.prepare(B)
    dA, dres = dg.dtensor(A), dg.dtensor(res)
    az = dg.dtensor(np.array([99], np.uint8))
    sa = dg.dtensor(np.array([0.02], np.float32))
    sb = dg.dtensor(np.array([0.003], np.float32))
    bias = dg.dtensor(rng.normal(0, 0.5, N).astype(np.float32))
    g = dg.dev.GemmArgs()
    g.M, g.N, g.K = M, N, K
    g.A, g.a_signed, g.B = dA.data_ptr, 0, pb
    g.a_zp, g.a_zp_len = az.data_ptr, 1
    g.sa, g.sb, g.sb_len, g.bias = sa.data_ptr, sb.data_ptr, 1, bias.data_ptr
    g.kernel_choice, g.epilogue = choice, dg.dev.EPI_DEQUANT
    Y0 = gpu.Tensor.device_empty((M, N), np.float32)
    g.Y = Y0.data_ptr
    dg.dev.gemm_i8(g, dg.stream)
    Y1 = gpu.Tensor.device_empty((M, N), np.float32)
    g.Y, g.residual = Y1.data_ptr, dres.data_ptr
    dg.dev.gemm_i8(g, dg.stream)
    y0, y1 = Y0.numpy(), Y1.numpy()
    gpu.synchronize()
    assert y1.tobytes() == (y0 + res).astype(np.float32).tobytes()


@pytest.mark.parametrize("seed", range(16))
def test_random_shapes_against_exact_products(gpu, seed):
    # Ragged shapes drawn at random around the tile sizes of the tensor-core
    # kernels (128 / 256 rows, 64..256 columns, whole and half tiles in the
    # last round, K not a multiple of the 128-byte K step): every output
    # element against the exact integer product (float64 holds it exactly).
    from gpu_util import DevGemm
    rng = np.random.default_rng(1000 + seed)
    M = int(rng.integers(130, 5200))
    N = int(rng.integers(70, 3100))
    K = 16 * int(rng.integers(1, 80))
    a_signed, b_signed = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
    A = rng.integers(-128 if a_signed else 0, 128 if a_signed else 256, (M, K)).astype(
        np.int8 if a_signed else np.uint8)
    B = rng.integers(-128 if b_signed else 0, 128 if b_signed else 256, (K, N)).astype(
        np.int8 if b_signed else np.uint8)
    za = int(rng.integers(-128 if a_signed else 0, 128 if a_signed else 256))
    dg = DevGemm(gpu)
    Y = dg.matmul_integer(A, B, za, None, 1)
    want = (A.astype(np.float64) - za) @ B.astype(np.float64)
    assert np.array_equal(Y.astype(np.float64), want), (M, N, K, a_signed, b_signed, za)


@pytest.mark.parametrize("seed", range(24))
def test_random_few_rows_long_k_auto_dispatch(gpu, seed):
    # The dispatcher's small-M territory at random: 1..600 rows, K up to 16384,
    # ragged N -- GEMV-shaped kernels (1..16 rows), split-K on single CTAs and
    # on CTA pairs (K >= 8192, few tiles), narrow tiles, the 2-CTA kernel at
    # three quarters occupancy.  Every output element against the exact integer
    # product (float64 holds it exactly), per-row A zero points included.
    from gpu_util import DevGemm
    rng = np.random.default_rng(2000 + seed)
    M = int(rng.choice([1, 2, 3, 7, 8, 15, 16, 17, 31, 64, 100, 128, 129, 200, 256, 300,
                        511, 512, 513, 600]))
    if seed % 3 == 0:
        M = int(rng.integers(1, 601))
    N = int(rng.integers(8, 3000))
    if seed % 2 == 0:
        N = (N + 3) & ~3
    K = 16 * int(rng.integers(1, 1025))
    if seed % 4 == 1:
        K = 16 * int(rng.integers(512, 1025))  # split-K territory
    a_signed, b_signed = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
    A = rng.integers(-128 if a_signed else 0, 128 if a_signed else 256, (M, K)).astype(
        np.int8 if a_signed else np.uint8)
    B = rng.integers(-128 if b_signed else 0, 128 if b_signed else 256, (K, N)).astype(
        np.int8 if b_signed else np.uint8)
    za = rng.integers(-128 if a_signed else 0, 128 if a_signed else 256,
                      M if seed % 5 == 0 else 1).astype(A.dtype)
    dg = DevGemm(gpu)
    Y = dg.matmul_integer(A, B, za, None, 0)
    want = (A.astype(np.float64) - za.astype(np.float64).reshape(-1, 1)) @ B.astype(np.float64)
    assert np.array_equal(Y.astype(np.float64), want), (M, N, K, a_signed, b_signed)

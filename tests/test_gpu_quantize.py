"""GPU parity: DynamicQuantizeLinear / QuantizeLinear / DequantizeLinear through
the C ABI against the CPU oracle.  Bit-exact for the uint8 tensor, the scale
and the zero point."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def check_dql(gpu, orc, x, device=False):
    want_y, want_s, want_z = orc.dynamic_quantize_linear(x)
    if device:
        y, s, z = gpu.dynamic_quantize_linear(x, device=True)
        y, s, z = y.numpy(), s.numpy(), z.numpy()
    else:
        y, s, z = gpu.dynamic_quantize_linear(x)
    assert s.tobytes() == want_s.tobytes(), (s, want_s)
    assert int(z) == int(want_z)
    assert y.shape == want_y.shape
    assert np.array_equal(y, want_y), np.flatnonzero(y.ravel() != want_y.ravel())[:10]


def test_config1_activation(gpu, orc):
    x = np.random.default_rng(42).normal(size=(128, 768)).astype(np.float32)
    check_dql(gpu, orc, x)
    check_dql(gpu, orc, x, device=True)


@pytest.mark.parametrize("n", [1, 2, 3, 5, 31, 33, 255, 1023, 1025, 4097, 100003])
def test_ragged_sizes(gpu, orc, n):
    x = np.random.default_rng(n).normal(0, 3, size=n).astype(np.float32)
    check_dql(gpu, orc, x)


def test_rank0_and_rank4(gpu, orc):
    check_dql(gpu, orc, np.array(2.5, np.float32))
    check_dql(gpu, orc, np.random.default_rng(1).normal(size=(2, 3, 5, 7)).astype(np.float32))


def test_edge_values(gpu, orc):
    check_dql(gpu, orc, np.zeros(1000, np.float32))                  # scale 0 -> NaN path
    check_dql(gpu, orc, np.linspace(1, 9, 777, dtype=np.float32))    # all positive
    check_dql(gpu, orc, -np.linspace(1, 9, 777, dtype=np.float32))   # all negative
    x = np.random.default_rng(3).normal(size=4099).astype(np.float32)
    x[[0, 100, 4098]] = np.nan
    check_dql(gpu, orc, x)                                           # NaN ignored by min/max
    x = np.random.default_rng(4).normal(size=513).astype(np.float32)
    x[7], x[9] = 1e30, -1e30
    check_dql(gpu, orc, x)                                           # huge range
    check_dql(gpu, orc, np.array([-0.0, 0.0, 1e-40, -1e-40, 1.0], np.float32))  # denormals


def test_exact_ties(gpu, orc):
    # range [-127.5, 127.5] -> scale 1.0, zero point 128 (127.5 rounds to even):
    # every k + 0.5 is an exact tie of x / scale.
    x = np.concatenate([np.arange(-127, 127, dtype=np.float32) + 0.5,
                        np.array([-127.5, 127.5], np.float32),
                        np.arange(-127, 128, dtype=np.float32)])
    _, s, _ = orc.dynamic_quantize_linear(x)
    assert s == 1.0
    check_dql(gpu, orc, x)


def test_values_crowded_around_ties(gpu, orc):
    # The kernel avoids the divide on its common path and falls back to the
    # exact divide near a rounding tie: crowd the input around ties, at every
    # magnitude of the quantized range and at offsets from far below to far
    # above the fallback threshold.
    rng = np.random.default_rng(9)
    for lo, hi in ((-3.7, 5.1), (-1000.0, 0.3), (-1e-3, 2e-3), (0.0, 7.77)):
        scale = np.float32((np.float32(hi) - np.float32(lo)) / np.float32(255))
        k = rng.integers(-300, 300, size=400000).astype(np.float32)
        off = rng.choice([0.0, 1e-7, -1e-7, 3e-6, -3e-6, 1e-4, -1e-4, 9e-4, -9e-4,
                          2e-3, -2e-3, 0.25], size=k.size).astype(np.float32)
        x = ((k + np.float32(0.5) + off) * scale).astype(np.float32)
        x = np.clip(x, np.float32(lo), np.float32(hi))
        x[0], x[1] = np.float32(lo), np.float32(hi)      # pins the range
        check_dql(gpu, orc, x)


def test_larger_than_l2(gpu, orc):
    # 48 Mi floats = 192 MiB > the 126 MB L2: the quantize pass re-reads HBM.
    x = np.random.default_rng(5).normal(size=48 * 1024 * 1024).astype(np.float32)
    check_dql(gpu, orc, x, device=True)


def test_repeated_calls_share_scratch(gpu, orc):
    rng = np.random.default_rng(6)
    for _ in range(5):
        check_dql(gpu, orc, rng.normal(0, rng.uniform(0.1, 10), size=70001).astype(np.float32),
                  device=True)


@pytest.mark.parametrize("signed", [False, True])
def test_quantize_linear(gpu, orc, signed):
    rng = np.random.default_rng(7)
    x = rng.normal(0, 40, size=(33, 129)).astype(np.float32)
    dt = np.int8 if signed else np.uint8
    zp = np.array(-3 if signed else 131, dt)
    want = orc.quantize(x, 0.37, float(zp), signed)
    got = gpu.quantize_linear(x, 0.37, zp, out_dtype=dt)
    assert np.array_equal(got, want)
    want = orc.quantize(x, 0.37, 0.0, signed)
    got = gpu.quantize_linear(x, 0.37, None, out_dtype=dt)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("dt", [np.uint8, np.int8, np.int32])
def test_dequantize_linear(gpu, orc, dt):
    rng = np.random.default_rng(8)
    info = np.iinfo(dt)
    x = rng.integers(max(info.min, -10**6), min(info.max, 10**6), size=(17, 65)).astype(dt)
    zp = np.array(5, dt)
    want = orc.dequantize_linear(x, 0.0123, 5)
    got = gpu.dequantize_linear(x, 0.0123, zp)
    assert got.tobytes() == want.tobytes()
    want = orc.dequantize_linear(x, 0.0123, 0)
    assert gpu.dequantize_linear(x, 0.0123, None).tobytes() == want.tobytes()


def test_argument_errors(gpu):
    with pytest.raises(gpu.OmcudaError) as ei:
        gpu.quantize_linear(np.ones((2, 3), np.float32), np.ones(3, np.float32))
    assert ei.value.code == gpu.ENOTSUP     # per-axis: rejected like the reference
    x = gpu.Tensor.from_numpy(np.ones(4, np.float32))
    y = gpu.Tensor.from_numpy(np.ones(5, np.uint8))
    s = gpu.Tensor.from_numpy(np.zeros((), np.float32))
    z = gpu.Tensor.from_numpy(np.zeros((), np.uint8))
    gpu.lib().omcudaDynamicQuantizeLinear(y.handle, s.handle, z.handle, x.handle)
    with pytest.raises(gpu.OmcudaError) as ei:
        gpu.check()
    assert ei.value.code == gpu.EINVAL

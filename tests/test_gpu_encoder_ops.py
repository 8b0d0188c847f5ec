"""GPU parity of the fp32 ops between the quantized linears of an encoder
graph.  Tolerance 1e-3 relative where a reduction is reordered (Softmax,
LayerNorm, MatMul, attention), 1e-5 for pointwise ops."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def close(got, want, rtol, atol):
    assert got.shape == want.shape
    assert np.allclose(got, want, rtol=rtol, atol=atol), np.abs(got - want).max()


@pytest.mark.parametrize("shape", [(7, 128), (3, 5, 33), (2, 12, 128, 128), (4, 1000)])
def test_softmax(gpu, orc, shape):
    x = np.random.default_rng(1).normal(0, 3, size=shape).astype(np.float32)
    close(gpu.softmax(x), orc.softmax(x), 1e-3, 1e-7)


@pytest.mark.parametrize("cols", [768, 1024, 100])
def test_layernorm(gpu, orc, cols):
    rng = np.random.default_rng(2)
    x = rng.normal(1, 2, size=(37, cols)).astype(np.float32)
    g, b = rng.normal(1, 0.1, cols).astype(np.float32), rng.normal(0, 0.1, cols).astype(np.float32)
    close(gpu.layer_normalization(x, g, b), orc.layernorm(x, g, b), 1e-3, 1e-5)
    close(gpu.layer_normalization(x, g, None), orc.layernorm(x, g, None), 1e-3, 1e-5)


def test_pointwise(gpu, orc):
    rng = np.random.default_rng(3)
    x = rng.normal(0, 2, size=(33, 257)).astype(np.float32)
    y = rng.normal(0, 2, size=(33, 257)).astype(np.float32)
    close(gpu.gelu(x), orc.gelu(x), 1e-5, 1e-7)
    assert gpu.add(x, y).tobytes() == (x + y).tobytes()
    t = rng.normal(size=(2, 5, 3, 16)).astype(np.float32)
    assert np.array_equal(gpu.transpose_0213(t), orc.transpose_0213(t))


def test_gelu_dense_sweep_relative_bound(gpu, orc):
    # 2 M points over [-8, 8].  The documented bound of omcudaGelu against the
    # reference's 0.5 x (1 + erff(x / sqrt 2)): 4e-6 relative and no absolute
    # term for x >= 0; for x < 0 additionally one rounding step of the
    # reference's own `1 + erff` (erff is rounded to fp32 before the add, which
    # quantizes the reference's result to multiples of 0.5 |x| 2^-24 -- the
    # library evaluates 0.5 x erfc(-x / sqrt 2) without that cancellation).
    x = np.linspace(-8.0, 8.0, 2 * 1024 * 1024 + 1).astype(np.float32)
    got, want = gpu.gelu(x).astype(np.float64), orc.gelu(x).astype(np.float64)
    x64 = x.astype(np.float64)
    err = np.abs(got - want)
    step = 0.5 * np.abs(x64) * 2.0 ** -24
    bound = 4e-6 * np.abs(want) + np.where(x < 0, step, 0.0)
    assert (err <= bound).all(), (x[np.argmax(err - bound)], (err / np.maximum(bound, 1e-300)).max())
    # purely relative, atol = 0, wherever the reference's quantization step is
    # below 1e-5 of its result (x >= -2.9), zero excluded
    sel = (x >= -2.9) & (want != 0)
    rel = err[sel] / np.abs(want[sel])
    assert rel.max() <= 1e-5, rel.max()
    # beyond x = -5.7 the reference is exactly -0; the library stays within
    # half a step of it
    far = x < -5.7
    assert (want[far] == 0).all() and (err[far] <= step[far]).all()
    print("\ngelu: max relative error for x >= -2.9: %.3g; max error / bound: %.3g"
          % (rel.max(), (err / np.maximum(bound, 1e-300)).max()))
    # special values
    sp = np.array([0.0, -0.0, np.inf, np.nan, 1e30, -1e30], np.float32)
    g = gpu.gelu(sp)
    assert g[0] == 0 and g[1] == 0 and g[2] == np.inf and np.isnan(g[3])
    assert g[4] == np.float32(1e30) and abs(g[5]) < 1e-7


def test_matmul_f32(gpu, orc):
    rng = np.random.default_rng(4)
    a = rng.normal(size=(3, 70, 65)).astype(np.float32)
    b = rng.normal(size=(3, 65, 50)).astype(np.float32)
    close(gpu.matmul_f32(a, b), orc.matmul_f32(a, b), 1e-3, 1e-4)
    b2 = rng.normal(size=(65, 20)).astype(np.float32)
    close(gpu.matmul_f32(a, b2), (a.reshape(-1, 65) @ b2).reshape(3, 70, 20), 1e-3, 1e-4)


@pytest.mark.parametrize("B,S,heads,dh", [(2, 128, 12, 64), (1, 77, 2, 64), (2, 40, 3, 32),
                                          (1, 512, 3, 64), (3, 256, 2, 64)])
def test_attention(gpu, orc, B, S, heads, dh):
    rng = np.random.default_rng(5)
    q, k, v = (rng.normal(size=(B, S, heads * dh)).astype(np.float32) for _ in range(3))
    scale = 1.0 / np.sqrt(dh)
    close(gpu.attention(q, k, v, heads, scale), orc.attention(q, k, v, heads, scale), 1e-3, 1e-5)


def test_attention_non_positive_scale(gpu, orc):
    # The graph's Mul constant may be any float.  The tensor-core kernel folds
    # the scale into the row maximum, which is only valid for a positive scale;
    # omcudaAttention sends every other value to the fp32 kernels (which scale
    # before taking the maximum), and the device-pointer entry of the
    # tensor-core kernel refuses it.
    from omcuda import dev
    rng = np.random.default_rng(19)
    B, S, heads, dh = 1, 128, 2, 64
    q, k, v = (rng.normal(size=(B, S, heads * dh)).astype(np.float32) for _ in range(3))
    for scale in (-0.125, 0.0):
        close(gpu.attention(q, k, v, heads, scale), orc.attention(q, k, v, heads, scale),
              1e-3, 1e-5)
    planes = gpu.Tensor.device_empty((2, B * S, 3 * heads * dh), np.uint16)
    out = gpu.Tensor.device_empty((B * S, heads * dh), np.float32)
    H = heads * dh
    for bad in (-0.125, 0.0, float("nan"), float("inf")):
        with pytest.raises(gpu.OmcudaError) as ei:
            dev.attention_bf16(planes.data_ptr, planes.data_ptr + 2 * B * S * 3 * H, 3 * H,
                               0, H, 2 * H, B, S, heads, dh, bad, out.data_ptr, H, None,
                               gpu.lib().omcudaGetStream())
        assert ei.value.code == gpu.EINVAL


@pytest.mark.parametrize("scales", [(0.1, 4.0, 0.1, 12.0), (6.0, 0.2, 0.2, 0.2),
                                    (0.5, 1.0, 2.0, 4.0)])
def test_attention_growing_and_shrinking_key_blocks(gpu, orc, scales):
    # The tcgen05 kernel keeps O in tensor memory and moves a row's exponent
    # offset only when a key block's maximum outgrows it by more than 2^8:
    # key blocks of very different magnitude make some rows move once, twice
    # or never, and make later blocks vanish against an early maximum.
    rng = np.random.default_rng(17)
    B, S, heads, dh = 2, 512, 2, 64
    q = rng.normal(0, 1.0, size=(B, S, heads * dh)).astype(np.float32)
    k = rng.normal(0, 1.0, size=(B, S, heads * dh)).astype(np.float32)
    v = rng.normal(0, 1.0, size=(B, S, heads * dh)).astype(np.float32)
    for j, f in enumerate(scales):
        k[:, 128 * j:128 * (j + 1)] *= np.float32(f)
    q[:, ::3] *= np.float32(0.05)        # rows whose scores stay small throughout
    scale = 1.0 / np.sqrt(dh)
    close(gpu.attention(q, k, v, heads, scale), orc.attention(q, k, v, heads, scale),
          1e-3, 1e-3)


def test_attention_peaked_scores(gpu, orc):
    # Head size 64 with a sequence that is a multiple of 128 runs on the
    # tcgen05 kernel; peaked scores (large logits) exercise the online
    # softmax's rescaling across key blocks.
    rng = np.random.default_rng(6)
    B, S, heads, dh = 2, 384, 2, 64
    q, k, v = (rng.normal(0, 2.5, size=(B, S, heads * dh)).astype(np.float32) for _ in range(3))
    scale = 1.0 / np.sqrt(dh)
    got = gpu.attention(q, k, v, heads, scale)
    # 1e-3 relative to the scale of the outputs (|v| reaches ~10 here): the
    # elementwise form would ask for 1e-8 absolute on outputs that cancel to 0.
    close(got, orc.attention(q, k, v, heads, scale), 1e-3, 1e-3)

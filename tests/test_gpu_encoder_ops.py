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
    close(gpu.gelu(x), orc.gelu(x), 1e-5, 1e-6)
    assert gpu.add(x, y).tobytes() == (x + y).tobytes()
    t = rng.normal(size=(2, 5, 3, 16)).astype(np.float32)
    assert np.array_equal(gpu.transpose_0213(t), orc.transpose_0213(t))


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

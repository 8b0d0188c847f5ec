"""GPU parity of the encoder harness (the run_main_graph of the BERT-shaped
configurations) against the CPU oracle's layer-by-layer restatement.

Three layers of evidence:
 1. the harness equals, bit for bit, the chain of individual library ops
    (DynamicQuantizeLinear, MatMulInteger + dequant, attention, Add,
    LayerNorm, Gelu) run one by one on the GPU -- so its fusions (one QKV
    GEMM, min/max folded into producers, Gelu in the GEMM epilogue, residual
    add inside LayerNorm) change nothing;
 2. each individual op is checked against the oracle elsewhere (bit-exact for
    the quantized ops, 1e-3 for the reordered fp32 reductions);
 3. end to end against the oracle the comparison can only be statistical: a
    one-ulp reordering difference in LayerNorm or attention can move an
    activation across a rounding boundary of the next DynamicQuantizeLinear,
    which changes that linear's input by one quantization step.  The rms
    deviation must stay below 1e-3 of the output's rms and the worst single
    deviation small."""
import numpy as np
import pytest

from omcuda.synthetic import make_encoder

pytestmark = pytest.mark.gpu


def oracle_encoder(orc, x, B, S, H, heads, F, layers):
    cur = x.reshape(B * S, H)
    for w in layers:
        cur = orc.encoder_layer(cur, B, S, H, heads, F, w)
    return cur.reshape(B, S, H)


def compare(got, want):
    """(rms error relative to the rms of the expected output, worst |error|)."""
    err = (got - want).astype(np.float64)
    rel_rms = float(np.sqrt((err ** 2).mean()) / np.sqrt((want.astype(np.float64) ** 2).mean()))
    return rel_rms, float(np.abs(err).max())


@pytest.mark.parametrize("B,S,H,heads,F,nl", [(2, 40, 128, 2, 256, 2),
                                              (1, 128, 768, 12, 3072, 1)])
def test_encoder_matches_oracle(gpu, orc, B, S, H, heads, F, nl):
    layers = make_encoder(7, H, F, nl)
    x = np.random.default_rng(8).normal(size=(B, S, H)).astype(np.float32)
    want = oracle_encoder(orc, x, B, S, H, heads, F, layers)
    enc = gpu.Encoder(H, heads, F, layers)
    got = enc.run(x)                      # host tensors, staged
    rel_rms, worst = compare(got, want)
    assert rel_rms < 1e-3 and worst < 5e-2, (rel_rms, worst)
    got_dev = enc.run(gpu.Tensor.from_numpy(x).to_device()).numpy()
    assert np.array_equal(got_dev, got)   # same kernels either way
    enc.close()


def unfused_layer_on_gpu(gpu, x, B, S, H, heads, w):
    """One encoder layer as separate library calls, everything on the device."""
    d = lambda a: gpu.Tensor.from_numpy(np.asarray(a)).to_device()
    X = d(x.reshape(B, S, H))

    def linear(inp, name, bias, i):
        return gpu.dyn_quant_linear(inp, d(w[name]), d(np.asarray(w["sc"][i], np.float32)),
                                    None, d(w[bias]), 0, device=True)
    q, k, v = linear(X, "wq", "bq", 0), linear(X, "wk", "bk", 1), linear(X, "wv", "bv", 2)
    ctx = gpu.attention(q, k, v, heads, 1.0 / np.sqrt(np.float32(H // heads)), device=True)
    a = linear(ctx, "wo", "bo", 3)
    h1 = gpu.layer_normalization(gpu.add(X, a, device=True), d(w["ln1g"]), d(w["ln1b"]),
                                 device=True)
    f = gpu.gelu(linear(h1, "w1", "b1", 4), device=True)
    o = linear(f, "w2", "b2", 5)
    y = gpu.layer_normalization(gpu.add(h1, o, device=True), d(w["ln2g"]), d(w["ln2b"]),
                                device=True)
    return y.numpy()


@pytest.mark.parametrize("B,S,H,heads,F,nl", [(2, 40, 128, 2, 256, 2),
                                              (2, 128, 768, 12, 3072, 2),
                                              # 64 MiB of activations: the residual
                                              # adds move into the GEMM tails
                                              (256, 512, 128, 2, 256, 1)])
def test_encoder_equals_unfused_chain_bit_exact(gpu, B, S, H, heads, F, nl):
    layers = make_encoder(12, H, F, nl)
    x = np.random.default_rng(13).normal(size=(B, S, H)).astype(np.float32)
    enc = gpu.Encoder(H, heads, F, layers)
    got = enc.run(x)
    cur = x
    for w in layers:
        cur = unfused_layer_on_gpu(gpu, cur, B, S, H, heads, w)
    assert got.tobytes() == cur.reshape(B, S, H).tobytes()
    enc.close()


def test_encoder_first_linear_is_bit_exact(gpu, orc):
    # Up to the first reduction-reordered op everything is integer or exactly
    # rounded fp32: the fused QKV projection must equal the oracle bit for bit.
    H, F = 128, 256
    layers = make_encoder(9, H, F, 1)
    w = layers[0]
    x = np.random.default_rng(10).normal(size=(3, 17, H)).astype(np.float32)
    for name, b, i in (("wq", "bq", 0), ("wk", "bk", 1), ("wv", "bv", 2)):
        want = orc.dyn_quant_linear(x, w[name], w["sc"][i], w[b])["Y"]
        got = gpu.dyn_quant_linear(x, w[name], w["sc"][i], None, w[b], 0)
        assert got.tobytes() == want.tobytes()


def test_pipelined_submit_equals_run_into(gpu):
    # Five different batches through the pipelined host-tensor calls (copies
    # of one call overlap the run of its neighbours, two staging slots) give,
    # bit for bit, what the synchronous call gives for each of them; nothing
    # is complete before wait(), everything after it.
    B, S, H, heads, F = 4, 128, 128, 2, 256
    layers = make_encoder(13, H, F, 2)
    enc = gpu.Encoder(H, heads, F, layers)
    rng = np.random.default_rng(14)
    # (seven batches over two staging slots: the first run of a slot goes
    # kernel by kernel, the second is captured as a CUDA graph, the later ones
    # replay it -- all must give the synchronous call's bytes)
    xs = [rng.normal(size=(B, S, H)).astype(np.float32) * (1 + i) for i in range(7)]
    want = []
    for x in xs:
        y = np.zeros((B, S, H), np.float32)
        enc.run_into(gpu.Tensor.from_numpy(x), gpu.Tensor.from_numpy(y))
        want.append(y)
    ys = [np.zeros((B, S, H), np.float32) for _ in xs]
    keep, counts = [], [gpu.launch_count()]
    for x, y in zip(xs, ys):
        tx, ty = gpu.Tensor.from_numpy(x), gpu.Tensor.from_numpy(y)
        keep.append((tx, ty))
        enc.submit(tx, ty)
        counts.append(gpu.launch_count())
    enc.wait()
    for y, w in zip(ys, want):
        assert np.array_equal(y, w)
    # a replayed run counts the launches it replays
    per_run = np.diff(counts)
    assert per_run[0] > 0 and (per_run == per_run[0]).all(), per_run
    # a larger batch afterwards grows the staging buffers
    x = rng.normal(size=(2 * B, S, H)).astype(np.float32)
    y, w = np.zeros_like(x), np.zeros_like(x)
    enc.run_into(gpu.Tensor.from_numpy(x), gpu.Tensor.from_numpy(w))
    tx, ty = gpu.Tensor.from_numpy(x), gpu.Tensor.from_numpy(y)
    enc.submit(tx, ty)
    enc.wait()
    assert np.array_equal(y, w)
    with pytest.raises(gpu.OmcudaError):
        enc.submit(gpu.Tensor.from_numpy(x).to_device(), gpu.Tensor.from_numpy(y))
    enc.close()


def test_replayed_runs_follow_the_quantization_mode(gpu):
    # The quantization mode is a process-wide setting that ends up in kernel
    # arguments: a run captured in one mode must not be replayed in another.
    B, S, H, heads, F = 2, 128, 128, 2, 256
    layers = make_encoder(17, H, F, 2)
    x = np.random.default_rng(18).normal(size=(B, S, H)).astype(np.float32)
    L = gpu.lib()
    enc = gpu.Encoder(H, heads, F, layers)
    tx = gpu.Tensor.from_numpy(x).to_device()
    ty = gpu.Tensor.device_empty((B, S, H), np.float32)
    try:
        for _ in range(4):          # kernel by kernel, captured, replayed twice
            enc.run_into(tx, ty)
        y_default = ty.numpy()
        L.omcudaSetQuantizationMode(1)  # OMCUDA_MODE_NO_ZERO_POINT
        enc.run_into(tx, ty)
        y_mode = ty.numpy()
        fresh = gpu.Encoder(H, heads, F, layers)
        want_mode = fresh.run(x)
        fresh.close()
        L.omcudaSetQuantizationMode(0)
        enc.run_into(tx, ty)
        y_back = ty.numpy()
    finally:
        L.omcudaSetQuantizationMode(0)
    enc.close()
    assert np.array_equal(y_mode, want_mode)
    assert not np.array_equal(y_mode, y_default)
    assert np.array_equal(y_back, y_default)


def test_encoder_rejects_wrong_input(gpu):
    layers = make_encoder(11, 128, 256, 1)
    enc = gpu.Encoder(128, 2, 256, layers)
    with pytest.raises(gpu.OmcudaError) as ei:
        enc.run(np.zeros((2, 8, 64), np.float32))
    assert ei.value.code == gpu.EINVAL
    enc.close()


def test_bert_large_size_batch_permutation(gpu):
    # Size-independent property at the full BERT-large-shaped configuration
    # (24 layers, hidden 1024, 16 heads, FFN 4096, batch 256 x 512 tokens):
    # the per-tensor ranges are order independent and every other op works on
    # one token or one sequence, so reversing the batch must reverse the
    # output bit for bit -- whatever CTA, tile or wave a sequence lands in.
    B, S, H, heads, F, nl = 256, 512, 1024, 16, 4096, 24
    layers = make_encoder(21, H, F, nl)
    enc = gpu.Encoder(H, heads, F, layers)
    rng = np.random.default_rng(22)
    x = rng.standard_normal((B, S, H), dtype=np.float32)
    y = enc.run(x)
    assert np.isfinite(y).all()
    y_rev = enc.run(np.ascontiguousarray(x[::-1]))
    assert np.array_equal(y_rev[::-1], y)
    # and the run is repeatable
    assert np.array_equal(enc.run(x), y)
    enc.close()

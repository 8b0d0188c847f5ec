"""Seeded synthetic weights for the BERT-shaped encoder configurations: every
Linear weight ~ N(0, 0.02) quantized per tensor, symmetric, to int8
(scale = max|W| / 127, round half even, clip to +-127); biases ~ N(0, 0.02);
LayerNorm gamma = 1 + N(0, 0.02), beta = N(0, 0.02)."""
import numpy as np


def quantize_weight(wf):
    scale = np.float32(np.abs(wf).max() / 127.0)
    q = np.clip(np.rint(wf / scale), -127, 127).astype(np.int8)
    return q, scale


def make_layer(rng, H, F):
    w = {}
    sc = []
    for name, shape in (("wq", (H, H)), ("wk", (H, H)), ("wv", (H, H)),
                        ("wo", (H, H)), ("w1", (H, F)), ("w2", (F, H))):
        q, s = quantize_weight(rng.normal(0, 0.02, shape).astype(np.float32))
        w[name] = q
        sc.append(s)
    w["sc"] = np.array(sc, np.float32)
    for name, n in (("bq", H), ("bk", H), ("bv", H), ("bo", H), ("b1", F), ("b2", H)):
        w[name] = rng.normal(0, 0.02, n).astype(np.float32)
    for g, b in (("ln1g", "ln1b"), ("ln2g", "ln2b")):
        w[g] = (1 + rng.normal(0, 0.02, H)).astype(np.float32)
        w[b] = rng.normal(0, 0.02, H).astype(np.float32)
    return w


def make_encoder(seed, H, F, layers):
    rng = np.random.default_rng(seed)
    return [make_layer(rng, H, F) for _ in range(layers)]

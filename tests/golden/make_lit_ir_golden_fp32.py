"""Generates tests/golden/lit_ir_golden_fp32.json: golden vectors for the fp32
ops of the encoder graphs (Softmax, MatMul, Gelu, LayerNormalization),
obtained by executing, with tests/golden/lit_ir_interp.py, the Krnl IR that
onnx-mlir's own lowering tests expect for them, on seeded inputs.

    python tests/golden/make_lit_ir_golden_fp32.py /path/to/onnx-mlir

Sources (paths in the onnx-mlir tree; the functions are named in the JSON):
  test/mlir/conversion/onnx_to_krnl/Math/Softmax_with_canonicalize.mlir
  test/mlir/conversion/onnx_to_krnl/Math/MatMul_with_canonicalize.mlir
  test/mlir/conversion/onnx_to_krnl/Math/Elementwise_with_canonicalize.mlir  (test_gelu_none)
  test/mlir/conversion/onnx_to_krnl/NN/Normalization_O3_SIMD_canonicalize.mlir
      (layernorm_4D_with_scale_bias_no_SIMD)
math.exp / math.erf are evaluated with the host libm, as a compiled model
does.  Tensors are stored as base64 of their little-endian float32 bytes.
The reference tree is needed only to regenerate; tests read the JSON.
"""
import base64
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from lit_ir_interp import extract_functions, run_lit_function  # noqa: E402

if len(sys.argv) < 2 and not os.environ.get("ONNX_MLIR_SRC"):
    sys.exit("usage: make_lit_ir_golden_fp32.py /path/to/onnx-mlir  (or set ONNX_MLIR_SRC)")
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ["ONNX_MLIR_SRC"]
BASE = os.path.join(REF, "test/mlir/conversion/onnx_to_krnl")
WANTED = [
    ("Math/Softmax_with_canonicalize.mlir", ["test_softmax_v11", "test_softmax_v13"]),
    ("Math/MatMul_with_canonicalize.mlir",
     ["test_matmul1", "test_matmul2", "test_matmul3", "test_matmul4", "test_matmul5",
      "test_matmul6"]),
    ("Math/Elementwise_with_canonicalize.mlir", ["test_gelu_none"]),
    ("NN/Normalization_O3_SIMD_canonicalize.mlir", ["layernorm_4D_with_scale_bias_no_SIMD"]),
]


def enc(a):
    a = np.ascontiguousarray(a, np.float32)
    return {"shape": list(a.shape), "f32_le_b64": base64.b64encode(a.tobytes()).decode()}


def make_input(rng, name, k, shape):
    if name == "test_gelu_none":
        # both tails, the region around the minimum, zero, large magnitudes
        v = np.array([-9, -6, -5, -4, -3.5, -3, -2.5, -2, -1.5, -1, -0.7518, -0.5, -0.1,
                      -1e-3, 0, 1e-3, 0.1, 0.5, 1, 2, 3, 4, 6, 9], np.float32)
        return v.reshape(shape)
    if name.startswith("test_softmax"):
        return rng.normal(0, 3.0, size=shape).astype(np.float32)
    if name.startswith("layernorm") and k == 0:
        return rng.normal(0.5, 2.0, size=shape).astype(np.float32)
    if name.startswith("layernorm"):
        return (rng.normal(1.0 if k == 1 else 0.0, 0.1, size=shape)).astype(np.float32)
    return rng.normal(size=shape).astype(np.float32)


def main():
    rng = np.random.default_rng(20240611)
    cases = []
    for rel, names in WANTED:
        funcs = extract_functions(open(os.path.join(BASE, rel)).read())
        for name in names:
            fn = funcs[name]
            params = [make_input(rng, name, k, [3 if d == "?" else int(d)
                                                for d in s.split("x") if d])
                      for k, (s, _) in enumerate(fn["params"])]
            it, ret = run_lit_function(fn["stmts"], [p.copy() for p in params], fn["maps"],
                                       fn["param_names"])
            out = np.asarray(it.env[ret[0]], np.float32)
            cases.append({"file": rel, "function": name,
                          "inputs": [enc(p) for p in params], "outputs": [enc(out)]})
            print("ok   %-40s %s" % (name, rel))
    doc = {"source": "onnx-mlir test/mlir/conversion/onnx_to_krnl (FileCheck "
                     "expectations executed by tests/golden/lit_ir_interp.py)",
           "generator": "tests/golden/make_lit_ir_golden_fp32.py", "cases": cases}
    out = os.path.join(HERE, "lit_ir_golden_fp32.json")
    with open(out, "w") as f:
        json.dump(doc, f)
    print("wrote %d cases, %d KiB" % (len(cases), os.path.getsize(out) // 1024))


if __name__ == "__main__":
    main()

"""Generates tests/golden/lit_ir_golden.json: golden vectors obtained by
executing, with tests/golden/lit_ir_interp.py, the Krnl IR that onnx-mlir's own
lowering tests expect for the quantized ops, on seeded inputs.

    python tests/golden/make_lit_ir_golden.py [/path/to/onnx-mlir]

Sources (paths in the onnx-mlir tree, functions named in the JSON):
  test/mlir/conversion/onnx_to_krnl/Quantization/DynamicQuantizeLinear_with_canonicalize.mlir
  test/mlir/conversion/onnx_to_krnl/Quantization/QuantizeLinear_with_canonicalize.mlir
  test/mlir/conversion/onnx_to_krnl/Quantization/DequantizeLinear_with_canonicalize.mlir
  test/mlir/conversion/onnx_to_krnl/Math/MatMulInteger_with_canonicalize.mlir
  test/mlir/conversion/onnx_to_krnl/Math/QLinearMatMul_with_canonicalize.mlir
The reference tree is needed only to regenerate; tests read the JSON.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from lit_ir_interp import _NP, extract_functions, run_lit_function  # noqa: E402

REF = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
BASE = os.path.join(REF, "test/mlir/conversion/onnx_to_krnl")
FILES = [
    "Quantization/DynamicQuantizeLinear_with_canonicalize.mlir",
    "Quantization/QuantizeLinear_with_canonicalize.mlir",
    "Quantization/DequantizeLinear_with_canonicalize.mlir",
    "Math/MatMulInteger_with_canonicalize.mlir",
    "Math/QLinearMatMul_with_canonicalize.mlir",
]


def make_input(rng, shape_s, ty, role, dyn):
    dims = [dyn if d == "?" else int(d) for d in shape_s.split("x") if d]
    if ty == "f32":
        if role == "scale":
            return np.array(rng.uniform(0.01, 0.2), np.float32).reshape(dims)
        x = rng.normal(0, 3.0, size=dims).astype(np.float32)
        if x.size >= 4:
            flat = x.reshape(-1)
            flat[0], flat[1] = np.float32(0.5) * 1, np.float32(-1.5)  # likely ties
        return x
    info = np.iinfo(_NP[ty])
    if role == "zp":
        lo, hi = (100, 150) if ty == "ui8" else (-20, 20)
        return rng.integers(lo, hi, size=dims).astype(_NP[ty])
    return rng.integers(info.min, int(info.max) + 1, size=dims).astype(_NP[ty])


def roles_for(func_name, n):
    if "dynamic_quantize" in func_name:
        return ["data"]
    if "qlinearmatmul" in func_name:
        return ["data", "scale", "zp", "data", "scale", "zp", "scale", "zp"]
    if "quantize" in func_name and "de" not in func_name:
        return ["data", "scale", "zp"][:n]
    if "dequantize" in func_name:
        return ["data", "scale", "zp"][:n]
    if "matmulinteger" in func_name:
        return ["data", "data", "zp", "zp"][:n]
    return ["data"] * n


def main():
    rng = np.random.default_rng(20240607)
    cases = []
    for rel in FILES:
        text = open(os.path.join(BASE, rel)).read()
        for name, fn in extract_functions(text).items():
            for rep, dyn in enumerate((5, 33)):
                roles = roles_for(name, len(fn["params"]))
                params = [make_input(rng, s, t, r, dyn)
                          for (s, t), r in zip(fn["params"], roles)]
                if "qlinearmatmul" in name:      # widen so that results wrap
                    params[1] = (params[1] * np.float32(4)).astype(np.float32)
                try:
                    it, ret = run_lit_function(fn["stmts"], [p.copy() for p in params],
                                               fn["maps"])
                except Exception as e:  # unsupported construct: report, skip
                    print("skip %s (%s: %s)" % (name, type(e).__name__, e))
                    break
                if "dynamic_quantize" in name:
                    outs = [it.env["%RES_"], it.env["%RES_1_"], it.env["%RES_2_"]]
                else:
                    outs = [it.env[r] for r in ret]
                cases.append({
                    "file": rel, "function": name,
                    "inputs": [{"dtype": p.dtype.name, "shape": list(p.shape),
                                "data": p.reshape(-1).tolist()} for p in params],
                    "outputs": [{"dtype": o.dtype.name, "shape": list(o.shape),
                                 "data": np.asarray(o).reshape(-1).tolist()}
                                for o in outs]})
                if not any("?" in s for s, _ in fn["params"]):
                    pass
            print("ok   %-40s %s" % (name, rel))
    doc = {"source": "onnx-mlir test/mlir/conversion/onnx_to_krnl (FileCheck "
                     "expectations executed by tests/golden/lit_ir_interp.py)",
           "generator": "tests/golden/make_lit_ir_golden.py", "cases": cases}
    out = os.path.join(HERE, "lit_ir_golden.json")
    with open(out, "w") as f:
        json.dump(doc, f)
    print("wrote %d cases, %d KiB" % (len(cases), os.path.getsize(out) // 1024))


if __name__ == "__main__":
    main()

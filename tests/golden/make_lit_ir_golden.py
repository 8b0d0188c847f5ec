"""Generates tests/golden/lit_ir_golden.json: golden vectors obtained by
executing, with tests/golden/lit_ir_interp.py, the Krnl IR that onnx-mlir's own
lowering tests expect for the quantized ops, on seeded inputs.

    python tests/golden/make_lit_ir_golden.py /path/to/onnx-mlir

(or ONNX_MLIR_SRC in the environment).  Also writes
tests/golden/lit_ir_golden_modes.json from the lowering tests of the two
non-default arithmetic modes:
  test/mlir/conversion/onnx_to_krnl/Quantization/QuantizationWithoutZeroPoint.mlir
      (--disable-quantization-zero-point)
  test/mlir/conversion/onnx_to_krnl/Quantization/QuantizeLinear_with_fast_math_canonicalize.mlir
      (convert-onnx-to-krnl=enable-fast-math)

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

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ONNX_MLIR_SRC")
if not REF or not os.path.isdir(REF):
    sys.exit("usage: make_lit_ir_golden.py /path/to/onnx-mlir  (or set ONNX_MLIR_SRC)")
BASE = os.path.join(REF, "test/mlir/conversion/onnx_to_krnl")
MODE_FILES = [   # (file, mode name)
    ("Quantization/QuantizationWithoutZeroPoint.mlir", "no_zero_point"),
    ("Quantization/QuantizeLinear_with_fast_math_canonicalize.mlir", "fast_math"),
]
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


def near_ties_that_tell_modes_apart(rng, x, scale):
    """Replaces most of x by values whose quotient x / scale and product
    x * RN(1 / scale) round to different integers, so that the fast-math
    fixture cannot be reproduced by the default arithmetic."""
    s = np.float32(scale.reshape(-1)[0])
    rcp = np.float32(1.0) / s
    found = []
    for k in rng.permutation(120):
        c = np.float32((np.float32(k) + np.float32(0.5)) * s)
        for step in range(-3, 4):
            v = c
            for _ in range(abs(step)):
                v = np.nextafter(v, np.float32(np.inf if step > 0 else -np.inf))
            if np.rint(np.float32(v / s)) != np.rint(np.float32(v * rcp)):
                found.append(np.float32(v))
                break
        if len(found) >= x.size - 2:
            break
    out = x.reshape(-1).copy()
    out[:len(found)] = found
    return out.reshape(x.shape)


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


def generate(files, seed, out_name):
    rng = np.random.default_rng(seed)
    cases = []
    for rel in files:
        mode = None
        if isinstance(rel, tuple):
            rel, mode = rel
        text = open(os.path.join(BASE, rel)).read()
        for name, fn in extract_functions(text).items():
            for rep, dyn in enumerate((5, 33)):
                roles = roles_for(name, len(fn["params"]))
                params = [make_input(rng, s, t, r, dyn)
                          for (s, t), r in zip(fn["params"], roles)]
                if mode == "fast_math":
                    params[0] = near_ties_that_tell_modes_apart(rng, params[0], params[1])
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
                    "file": rel, "function": name, "mode": mode,
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
    out = os.path.join(HERE, out_name)
    with open(out, "w") as f:
        json.dump(doc, f)
    print("wrote %d cases, %d KiB" % (len(cases), os.path.getsize(out) // 1024))


def main():
    generate(FILES, 20240607, "lit_ir_golden.json")
    generate(MODE_FILES, 20240612, "lit_ir_golden_modes.json")


if __name__ == "__main__":
    main()

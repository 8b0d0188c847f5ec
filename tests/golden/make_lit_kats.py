"""Extracts known-answer vectors for the quantized path from onnx-mlir's own
lit tests and writes them to lit_kats.json (committed beside this script).

    python tests/golden/make_lit_kats.py /path/to/onnx-mlir      (or ONNX_MLIR_SRC)

Source: test/mlir/onnx/onnx_constprop.mlir.  Its constant-propagation tests
fold MatMulInteger and Round on literal operands and FileCheck the folded
constant, so each test function is an (inputs, expected output) pair held by
the reference itself.  Only functions whose operands are all literal constants
and whose CHECK line pins a value are taken; functions with a runtime argument
(the *_zero cases, whose result does not depend on the argument) are skipped so
that every vector is literal.

The reference tree is only needed to regenerate the file; tests read the JSON.
"""
import json
import os
import re
import sys

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ONNX_MLIR_SRC")
if not REF or not os.path.isdir(REF):
    sys.exit("usage: make_lit_kats.py /path/to/onnx-mlir  (or set ONNX_MLIR_SRC)")
SRC = os.path.join(REF, "test/mlir/onnx/onnx_constprop.mlir")
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lit_kats.json")

TYPE_RE = re.compile(r"tensor<((?:\d+x)*)(ui8|i8|i32|f32)>")


def parse_dense(text):
    """dense<...> payload -> nested python list or scalar."""
    text = text.strip()
    # MLIR literal syntax for these cases is JSON-compatible.
    return json.loads(text)


def shape_of(tstr):
    m = TYPE_RE.search(tstr)
    dims = [int(d) for d in m.group(1).split("x") if d]
    return dims, m.group(2)


def flatten(v):
    if isinstance(v, list):
        out = []
        for e in v:
            out += flatten(e)
        return out
    return [v]


def expand(value, dims):
    n = 1
    for d in dims:
        n *= d
    flat = flatten(value)
    if len(flat) == 1 and n != 1:
        flat = flat * n  # splat
    assert len(flat) == n, (value, dims)
    return flat


CONST_RE = re.compile(
    r"(%\w+)\s*=\s*\"?onnx\.Constant\"?\(?\)?\s*(?:\{value\s*=\s*)?dense<(.+?)>\s*:\s*(tensor<[^>]*>)")
NOVALUE_RE = re.compile(r"(%\w+)\s*=\s*\"onnx\.NoValue\"")
MMI_RE = re.compile(
    r"\"onnx\.MatMulInteger\"\(([^)]*)\)\s*:\s*\(([^)]*)\)\s*->\s*(tensor<[^>]*>)")
ROUND_RE = re.compile(r"\"onnx\.Round\"\((%\w+)\)")
CHECK_CONST_RE = re.compile(
    r"//\s*CHECK:.*onnx\.Constant dense<(.+)>\s*:\s*(tensor<[^>]*>)")


def clean_check(payload):
    # FileCheck escapes a leading "[[" as {{\[}}[ and "]]" as ]{{\]}}.
    return payload.replace("{{\\[}}", "[").replace("{{\\]}}", "]")


def main():
    text = open(SRC).read()
    blocks = text.split("// -----")
    kats = []
    for blk in blocks:
        m = re.search(r"func\.func @(\w+)\(([^)]*)\)", blk)
        if not m:
            continue
        name, args = m.group(1), m.group(2).strip()
        if args:
            continue  # has runtime arguments: not a literal vector
        consts = {}
        for cm in CONST_RE.finditer(blk):
            if not TYPE_RE.search(cm.group(3)):
                continue  # element type outside this path
            try:
                parse_dense(cm.group(2))
            except ValueError:
                continue  # hex / opaque literal
            dims, dt = shape_of(cm.group(3))
            consts[cm.group(1)] = {
                "shape": dims, "dtype": dt,
                "data": expand(parse_dense(cm.group(2)), dims)}
        for nm in NOVALUE_RE.finditer(blk):
            consts[nm.group(1)] = None
        chk = CHECK_CONST_RE.search(blk)
        if not chk or not TYPE_RE.search(chk.group(2)):
            continue
        if not (MMI_RE.search(blk) or name == "test_round"):
            continue
        edims, edt = shape_of(chk.group(2))
        expected = {"shape": edims, "dtype": edt,
                    "data": expand(parse_dense(clean_check(chk.group(1))), edims)}
        mm = MMI_RE.search(blk)
        if mm:
            ops = [o.strip() for o in mm.group(1).split(",")]
            if any(o not in consts for o in ops):
                continue
            kats.append({"name": name, "op": "MatMulInteger",
                         "A": consts[ops[0]], "B": consts[ops[1]],
                         "a_zero_point": consts[ops[2]],
                         "b_zero_point": consts[ops[3]],
                         "expected": expected})
            continue
        rm = ROUND_RE.search(blk)
        if rm and rm.group(1) in consts and name == "test_round":
            kats.append({"name": name, "op": "Round",
                         "X": consts[rm.group(1)], "expected": expected})
    doc = {
        "source": "onnx-mlir test/mlir/onnx/onnx_constprop.mlir",
        "generator": "tests/golden/make_lit_kats.py",
        "cases": kats,
    }
    with open(OUT, "w") as f:
        json.dump(doc, f, indent=1)
    print("wrote %d cases to %s" % (len(kats), OUT))
    for k in kats:
        print("  ", k["op"], k["name"])


if __name__ == "__main__":
    main()

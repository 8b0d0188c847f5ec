"""The compiler plugin under plugin/ (an onnx-mlir accelerator laid out like
src/Accelerators/NNPA) cannot be compiled without LLVM/MLIR.  What can be
checked without it: every krnl.call the plugin emits -- the table its patterns
are generated from, the onnx.Custom calls of its rewrites, the expected lines
of its lit tests and the LLVM-level calls of its allocation pass -- names a
function that include/omcuda.h declares with exactly that many tensor and
scalar parameters and that libomcuda.so exports; and the accelerator class
overrides every pure virtual the framework declares."""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLUGIN = os.path.join(ROOT, "plugin")
ACCEL = os.path.join(PLUGIN, "src", "Accelerators", "CUDA")


def header_prototypes():
    """{name: (tensor params, int64 params, double params)} of omcuda.h."""
    text = open(os.path.join(ROOT, "include", "omcuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = {}
    for m in re.finditer(r"\b(\w+)\s*\(([^()]*)\)\s*;", text):
        name, params = m.group(1), m.group(2)
        ps = [p.strip() for p in params.split(",") if p.strip() and p.strip() != "void"]
        protos[name] = (sum("OMTensor *" in p for p in ps),
                        sum(p.startswith("int64_t") for p in ps),
                        sum(p.startswith("double") for p in ps), ps)
    return protos


def table_calls():
    """(function, results, operands, attribute names) per line of the table."""
    text = open(os.path.join(ACCEL, "Conversion", "ONNXToKrnl", "OMCUDACalls.inc")).read()
    out = []
    for m in re.finditer(r'^OMCUDA_CALL\(\s*\w+,\s*\w+,\s*"(\w+)",\s*(\d+),\s*(\d+),\s*"([^"]*)"\)',
                         text, flags=re.M):
        out.append((m.group(1), int(m.group(2)), int(m.group(3)),
                    [a for a in m.group(4).split(",") if a]))
    for m in re.finditer(r'^OMCUDA_CUSTOM_CALL\(\s*"(\w+)",\s*(\d+),\s*(\d+),\s*"([^"]*)"\)',
                         text, flags=re.M):
        out.append((m.group(1), int(m.group(2)), int(m.group(3)),
                    [a for a in m.group(4).split(",") if a]))
    return out


def lit_calls():
    """(file, function, results, parameter types, attributes) of every
    "krnl.call" line the lit tests expect."""
    out = []
    pat = re.compile(r'"krnl\.call"\((.*?)\) <\{funcName = "(\w+)", numOfOutput = (\d+) : si64\}>'
                     r'(?: \{(.*?)\})? : \((.*?)\) -> \(\)')
    for path in glob.glob(os.path.join(PLUGIN, "test", "mlir", "accelerators", "cuda", "**",
                                       "*.mlir"), recursive=True):
        for line in open(path):
            if "CHECK" not in line:
                continue
            m = pat.search(line)
            if m:
                types = re.findall(r"memref<[^>]*>|none|\bf32\b|\bi64\b", m.group(5))
                attrs = [a.split("=")[0].strip() for a in (m.group(4) or "").split(",") if a.strip()]
                out.append((os.path.basename(path), m.group(2), int(m.group(3)), types, attrs))
    return out


def exported():
    return ctypes.CDLL(os.path.join(ROOT, "onnx-mlir_b200", "lib", "libomcuda.so"))


def test_every_table_entry_matches_the_header_and_the_library(built):
    protos, lib = header_prototypes(), exported()
    calls = table_calls()
    assert len(calls) >= 13
    for func, nres, nops, attrs in calls:
        assert func in protos, func
        tensors, ints, doubles, ps = protos[func]
        assert tensors == nres + nops, (func, ps)
        assert ints + doubles == len(attrs), (func, ps)
        # krnl.call passes attributes in name order: the header's scalar
        # parameters must be named (and therefore ordered) the same way
        scalars = [p.split()[-1] for p in ps if not "OMTensor" in p]
        assert scalars == sorted(attrs) == attrs, (func, scalars, attrs)
        assert hasattr(lib, func), func


def test_every_expected_krnl_call_line_matches_the_header(built):
    protos, lib = header_prototypes(), exported()
    table = {f: (r, o, a) for f, r, o, a in table_calls()}
    calls = lit_calls()
    assert len(calls) >= 14
    for fname, func, nres, types, attrs in calls:
        assert func in protos and func in table, (fname, func)
        tensors, ints, doubles, ps = protos[func]
        assert nres == table[func][0], (fname, func)
        assert len(types) == tensors, (fname, func, types, ps)
        assert all(t.startswith("memref") or t == "none" for t in types), (fname, func)
        assert attrs == table[func][2], (fname, func, attrs)
        assert hasattr(lib, func)
    # every function of the table is exercised by at least one lit line
    assert {c[1] for c in calls} == set(table)


def test_rewrites_and_allocation_pass_name_exported_functions(built):
    lib = exported()
    fuse = open(os.path.join(ACCEL, "Transform", "ONNX", "FuseDynQuantLinear.cpp")).read()
    names = set(re.findall(r'getStringAttr\("(omcuda\w+)"\)', fuse))
    assert names == {"omcudaDynQuantLinear"}
    alloc = open(os.path.join(ACCEL, "Transform", "ReplaceMallocByDeviceAlloc.cpp")).read()
    for fn in re.findall(r'call\(\{[^}]*\}, "(\w+)"', alloc):
        assert fn.startswith("omcuda") and hasattr(lib, fn), fn
    # the runtime hooks the generated entry point calls for an accelerator named CUDA
    for fn in ("OMInitAccelCUDA", "OMInitCompatibleAccelCUDA", "OMShutdownAccelCUDA"):
        assert hasattr(lib, fn)
    assert ctypes.c_long.in_dll(lib, "OMIsInitAccelCUDA") is not None
    acc = open(os.path.join(ACCEL, "CUDAAccelerator.cpp")).read()
    assert 'addCompilerConfig(CCM_SHARED_LIB_DEPS, {"omcuda"}' in acc
    assert "Accelerator *createCUDA()" in acc


def test_accelerator_overrides_every_pure_virtual():
    # The pure virtuals of onnx_mlir::accel::Accelerator
    # (src/Accelerators/Accelerator.hpp:61-176 of onnx-mlir).
    pure = ["getVersionNumber", "addPasses", "registerDialects", "registerPasses",
            "configurePasses", "convertTensorTypeToMemRefType", "conversionTargetONNXToKrnl",
            "rewritePatternONNXToKrnl", "conversionTargetKrnlToLLVM", "rewritePatternKrnlToLLVM"]
    hpp = open(os.path.join(ACCEL, "CUDAAccelerator.hpp")).read()
    cpp = open(os.path.join(ACCEL, "CUDAAccelerator.cpp")).read()
    for name in pure:
        assert re.search(r"\b%s\(" % name, hpp), name
        assert re.search(r"CUDAAccelerator::%s\(" % name, cpp), name
    opts = open(os.path.join(ACCEL, "Compiler", "CUDACompilerOptions.hpp")).read()
    for macro in ("INSTRUMENTSTAGE_ENUM_CUDA", "INSTRUMENTSTAGE_CL_ENUM_CUDA",
                  "PROFILEIR_CL_ENUM_CUDA", "OPTREPORT_ENUM_CUDA", "OPTREPORT_CL_ENUM_CUDA"):
        assert re.search(r"#define %s\b" % macro, opts), macro
    # every source the cmake file lists exists
    cm = open(os.path.join(ACCEL, "CMakeLists.txt")).read()
    for src in re.findall(r"^\s+([\w/]+\.cpp)\s*$", cm, flags=re.M):
        assert os.path.exists(os.path.join(ACCEL, src)), src


def test_backend_test_list_names_exported_symbols_of_lowered_ops(built):
    # plugin/test/accelerators/CUDA/backend/CMakeLists.txt lists, per ONNX
    # backend node test, the library function the compiled model must refer to
    # (the instruction check of test/accelerators/NNPA/backend).  Every symbol
    # must be a krnl.call target of the call table and an export of the
    # library; every listed test must belong to an op with a table entry.
    lib = exported()
    table = {c[0] for c in table_calls()}
    src = open(os.path.join(PLUGIN, "test", "accelerators", "CUDA", "backend",
                            "CMakeLists.txt")).read()
    body = src[src.index("set(CUDA_TEST_LIST"):]
    body = body[:body.index("\n)\n")]
    entries = re.findall(r'^\s*(test_\w+),(\w+),("[^"]*"|NO_DYNAMIC_SHAPE_TEST)\s*$', body, re.M)
    assert len(entries) >= 15
    for test, symbol, dims in entries:
        assert symbol in table, (test, symbol)
        assert hasattr(lib, symbol), symbol
        op = symbol[len("omcuda"):].lower()
        assert op.replace("normalization", "_normalization") in test or op in test.replace("_", ""), \
            (test, symbol)
    # the ops of the quantized path are all there
    assert {"omcudaDynamicQuantizeLinear", "omcudaQuantizeLinear", "omcudaDequantizeLinear",
            "omcudaMatMulInteger", "omcudaQLinearMatMul"} <= {e[1] for e in entries}
    num = open(os.path.join(PLUGIN, "test", "accelerators", "CUDA", "numerical",
                            "CMakeLists.txt")).read()
    for symbol in re.findall(r"^add_cuda_numerical_test\(Test\w+ (\w+)", num, re.M):
        assert symbol in table and hasattr(lib, symbol), symbol

"""Builds libomcuda (sm_100a) and the CPU oracle in-tree.

    python onnx-mlir_b200/build.py [--force]

Outputs:
    onnx-mlir_b200/lib/libomcuda.so   the product: CUDA kernels + C ABI
    oracle/_build/liboracle.so        test infrastructure: CPU restatement
    oracle/_ref/libcruntime_ref.so    only where the onnx-mlir tree is present:
                                      the reference's own OMTensor runtime,
                                      compiled from its sources where they lie,
                                      used to check ABI compatibility
nvcc cross-compiles without a GPU, so this runs on a CPU-only machine.
"""
import concurrent.futures
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "lib", "obj")
LIB = os.path.join(LIBDIR, "libomcuda.so")

SOURCES = [
    "runtime/om_tensor.c",
    "runtime/context.cpp",
    "runtime/execution_session.cpp",
    "api/krnl_call_api.cpp",
    "api/no_alloc.cu",
    "model/encoder.cpp",
    "kernels/dql.cu",
    "kernels/gemm_simt.cu",
    "kernels/gemm_tc.cu",
    "kernels/encoder_ops.cu",
    "kernels/attention_mma.cu",
    "kernels/attention_tc.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo",
    # The reference never contracts mul+add into fma; neither may nvcc.
    "-fmad=false",
    "-Xcompiler", "-fPIC",
    "-I", os.path.join(ROOT, "include"),
    "-I", CSRC,
]


def _newer(src_paths, out):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in src_paths)


def _headers():
    hs = []
    for base in (CSRC, os.path.join(ROOT, "include")):
        for d, _, fs in os.walk(base):
            hs += [os.path.join(d, f) for f in fs if f.endswith((".h", ".cuh"))]
    return hs


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + cmd[0])
    return r.stdout + r.stderr


def build_lib(force=False, verbose=False):
    os.makedirs(OBJDIR, exist_ok=True)
    headers = _headers()
    jobs = []
    objs = []
    for rel in SOURCES:
        src = os.path.join(CSRC, rel)
        if not os.path.exists(src):
            continue
        obj = os.path.join(OBJDIR, rel.replace("/", "_") + ".o")
        objs.append(obj)
        if force or _newer([src] + headers, obj):
            cmd = ["nvcc"] + NVCC_FLAGS
            if src.endswith(".cpp"):
                cmd += ["-x", "cu"]
            if verbose:
                cmd += ["-Xptxas", "-v"]
            cmd += ["-c", src, "-o", obj]
            jobs.append(cmd)
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        outs = list(ex.map(_run, jobs))
    if verbose:
        for o in outs:
            sys.stderr.write(o)
    if jobs or not os.path.exists(LIB):
        _run(["nvcc", "-shared", "-cudart", "static", "-o", LIB] + objs +
             ["-Xcompiler", "-fPIC", "-lpthread", "-ldl"])
    return LIB


def build_oracle(force=False):
    odir = os.path.join(ROOT, "oracle")
    out = os.path.join(odir, "_build", "liboracle.so")
    srcs = [os.path.join(odir, "oracle.c"), os.path.join(odir, "oracle.h")]
    if force or _newer(srcs, out):
        _run(["make", "-s", "-C", odir, "oracle"])
    return out


def build_ref_runtime(force=False):
    """Compiles the reference's OMTensor runtime where its tree is present."""
    odir = os.path.join(ROOT, "oracle")
    ref = os.environ.get("ONNX_MLIR_SRC", "/root/reference")
    out = os.path.join(odir, "_ref", "libcruntime_ref.so")
    if not os.path.isdir(os.path.join(ref, "src", "Runtime")):
        return out if os.path.exists(out) else None
    if force or not os.path.exists(out):
        _run(["make", "-s", "-C", odir, "ref", "ONNX_MLIR_SRC=" + ref])
    return out


def build_all(force=False, verbose=False):
    lib = build_lib(force, verbose)
    orc = build_oracle(force)
    ref = build_ref_runtime(force)
    return lib, orc, ref


if __name__ == "__main__":
    force = "--force" in sys.argv
    verbose = "-v" in sys.argv
    for p in build_all(force, verbose):
        print(p)

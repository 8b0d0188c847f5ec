"""Builds libomcuda (sm_100a) in-tree.

    python onnx-mlir_b200/build.py [--force] [-v]

Output: onnx-mlir_b200/lib/libomcuda.so, the product (CUDA kernels + C ABI).
nvcc cross-compiles without a GPU, so this runs on a CPU-only machine.  (The
test infrastructure -- the CPU oracle -- has its own script, oracle/build.py.)
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


if __name__ == "__main__":
    print(build_lib("--force" in sys.argv, "-v" in sys.argv))

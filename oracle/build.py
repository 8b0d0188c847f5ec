"""Builds the test infrastructure under oracle/: the CPU oracle, and -- where
the onnx-mlir source tree is present -- the reference's own OMTensor runtime,
compiled from its sources where they lie (used to check ABI compatibility).

    python oracle/build.py [--force]

Outputs:
    oracle/_build/liboracle.so
    oracle/_ref/libcruntime_ref.so    (only with the onnx-mlir tree: ONNX_MLIR_SRC,
                                       else a checkout named `reference` next to
                                       this repository)
"""
import os
import subprocess
import sys

ODIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(ODIR)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + cmd[0])


def _newer(srcs, out):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in srcs)


def build_oracle(force=False):
    out = os.path.join(ODIR, "_build", "liboracle.so")
    srcs = [os.path.join(ODIR, "oracle.c"), os.path.join(ODIR, "oracle.h")]
    if force or _newer(srcs, out):
        _run(["make", "-s", "-C", ODIR, "oracle"])
    return out


def build_ref_runtime(force=False):
    """Compiles the reference's OMTensor runtime where its tree is present."""
    ref = os.environ.get("ONNX_MLIR_SRC") or os.path.join(os.path.dirname(ROOT), "reference")
    out = os.path.join(ODIR, "_ref", "libcruntime_ref.so")
    if not os.path.isdir(os.path.join(ref, "src", "Runtime")):
        return out if os.path.exists(out) else None
    if force or not os.path.exists(out):
        _run(["make", "-s", "-C", ODIR, "ref", "ONNX_MLIR_SRC=" + ref])
    return out


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_ref_runtime(force))

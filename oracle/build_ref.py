"""Compile the reference project's own CUDA kernels, in place, for sm_100a.

Test infrastructure only.  The sources are NOT copied: nvcc reads
``<reference>/kernels/*.cu`` where they lie and writes one shared library,
``oracle/_ref/libref_kernels.so`` (git-ignored), together with the thin
``extern "C"`` doors of ``oracle/ref_shim.cu``.  The library lets the GPU tests
and the benchmark run the unmodified reference kernels (its sm_80-era
mma.sync / dp4a code, recompiled) beside the new ones on the same B200.

The reference checkout is looked for in ``$I8TK_REFERENCE_DIR``, else in a
directory named ``reference`` next to this repository.  When it is absent
(e.g. on a machine that only received the built files) nothing is built and
whatever library is already there is used.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libref_kernels.so")
KERNELS = ["int8_decode_attention.cu", "int8_mlp.cu", "int8_attention.cu", "quant_utils.cu"]


def reference_dir():
    d = os.environ.get("I8TK_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    return d if os.path.isdir(os.path.join(d, "kernels")) else None


def build(force=False):
    ref = reference_dir()
    if ref is None:
        return LIB if os.path.exists(LIB) else None
    srcs = [os.path.join(ref, "kernels", k) for k in KERNELS] + [os.path.join(HERE, "ref_shim.cu")]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(s) <= os.path.getmtime(LIB) for s in srcs):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--std=c++17", "-shared",
           "-Xcompiler", "-fPIC", "-o", LIB] + srcs
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))

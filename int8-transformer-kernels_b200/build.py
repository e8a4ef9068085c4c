"""In-tree build of the native code (no JIT cache, no install step).

Produces, beside this file:
  libi8tk.so  -- the C-ABI CUDA library (include/i8tk.h), nvcc, sm_100a only
  libi8tk_compat.so -- the reference's C++-linkage launchers over it (include/i8tk_compat.h)
  int8_ext*.so -- the PyTorch binding over it (pybind11, no kernels)
  build/compat_driver -- torch-free program that links the compat launchers by their C++ names
                         (source: tests/compat_driver.cpp; built only when that file is present)

``python build.py`` builds what is out of date; ``build_all(force=True)``
rebuilds everything.  nvcc cross-compiles without a GPU.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libi8tk.so")
COMPAT_LIB = os.path.join(HERE, "libi8tk_compat.so")
COMPAT_DRIVER = os.path.join(HERE, "build", "compat_driver")
COMPAT_DRIVER_SRC = os.path.join(ROOT, "tests", "compat_driver.cpp")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
              "-std=c++17", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _cu_sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps(extra=()):
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(ROOT, "include", "i8tk.h"))
    deps.extend(extra)
    return deps


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd):
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def ext_path():
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(HERE, "int8_ext" + suffix)


def build_lib(force=False, verbose_ptxas=False):
    if not force and not _stale(LIB, _deps()):
        return LIB
    objs = []
    for src in _cu_sources():
        obj = os.path.join(HERE, "build", os.path.basename(src) + ".o")
        os.makedirs(os.path.dirname(obj), exist_ok=True)
        cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose_ptxas else []) + \
              ["-c", src, "-o", obj]
        _run(cmd)
        objs.append(obj)
    _run(["nvcc", "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"])
    return LIB


def build_ext(force=False):
    target = ext_path()
    if not force and not _stale(target, _deps([LIB])):
        return target
    import torch
    from torch.utils import cpp_extension
    inc = cpp_extension.include_paths(device_type="cuda")
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared",
           "-DTORCH_EXTENSION_NAME=int8_ext", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I" + sysconfig.get_paths()["include"]]
    cmd += ["-I" + p for p in inc]
    cmd += [os.path.join(CSRC, "int8_ext.cpp"), "-o", target,
            "-L" + HERE, "-li8tk", "-Wl,-rpath,$ORIGIN",
            "-L" + torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            "-ltorch_python", "-Wl,-rpath," + torch_lib]
    _run(cmd)
    return target


def build_compat(force=False):
    """The reference's native launchers (C++ linkage) as a thin library over libi8tk.so."""
    src = os.path.join(CSRC, "compat_launchers.cpp")
    hdr = os.path.join(ROOT, "include", "i8tk_compat.h")
    if force or _stale(COMPAT_LIB, [src, hdr, LIB, os.path.join(ROOT, "include", "i8tk.h")]):
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-I" + os.path.join(CUDA_HOME, "include"), src,
              "-o", COMPAT_LIB, "-L" + HERE, "-li8tk", "-L" + os.path.join(CUDA_HOME, "lib64"), "-lcudart",
              "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(CUDA_HOME, "lib64")])
    if os.path.exists(COMPAT_DRIVER_SRC) and (force or _stale(COMPAT_DRIVER, [COMPAT_DRIVER_SRC, COMPAT_LIB, hdr])):
        os.makedirs(os.path.dirname(COMPAT_DRIVER), exist_ok=True)
        _run(["g++", "-O2", "-std=c++17", "-I" + os.path.join(CUDA_HOME, "include"), COMPAT_DRIVER_SRC,
              "-o", COMPAT_DRIVER, "-L" + HERE, "-li8tk_compat", "-li8tk",
              "-L" + os.path.join(CUDA_HOME, "lib64"), "-lcudart",
              "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath," + os.path.join(CUDA_HOME, "lib64")])
    return COMPAT_LIB


def build_all(force=False):
    build_lib(force)
    build_compat(force)
    build_ext(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)

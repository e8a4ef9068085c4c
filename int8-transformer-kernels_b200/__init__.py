"""B200 (sm_100a) INT8 decode-attention / quantiser / fused-MLP kernels.

Host-side mirror of the reference's ``int8_ext`` torch extension
(``kernels/int8_ext.cu:458-479``) over a C-ABI CUDA library
(``include/i8tk.h``).  The directory name is not a Python identifier; load it
with ``importlib.import_module("int8-transformer-kernels_b200")``.

  ``int8_ext``   the compiled binding: same op names / signatures as the reference
  ``cabi``       ctypes view of the raw C ABI (status codes, workspace queries)
  ``sharding``   multi-GPU helpers: (batch, head) sharding and KV-sequence sharding
  ``block``      a pre-LN transformer block around the ops (the caller either side of the path)

There is no CPU or eager fallback: importing ``int8_ext`` raises if the native
libraries have not been built (``python build.py`` in this directory).
"""
import importlib
import importlib.util
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))


def _load_ext():
    from . import build as _build
    path = _build.ext_path()
    if not os.path.exists(path) or not os.path.exists(_build.LIB):
        raise ImportError(
            "native libraries missing: run `python build.py` in %s (nvcc, sm_100a); "
            "there is no fallback path" % _HERE)
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    spec = importlib.util.spec_from_file_location("int8_ext", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules.setdefault("int8_ext", mod)
    return mod


def __getattr__(name):
    if name == "int8_ext":
        mod = _load_ext()
        globals()["int8_ext"] = mod
        return mod
    if name in ("cabi", "sharding", "block"):
        mod = importlib.import_module("." + name, __name__)
        globals()[name] = mod
        return mod
    raise AttributeError(name)

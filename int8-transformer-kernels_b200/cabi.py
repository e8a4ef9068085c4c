"""ctypes view of the C ABI declared in ``include/i8tk.h``.

Used where a caller has raw device pointers rather than torch tensors, and by
the tests to check status codes and that every declared symbol is exported.
``load()`` raises if ``libi8tk.so`` is missing -- there is no fallback.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libi8tk.so")

OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_UNSUPPORTED = 2
ERR_WORKSPACE = 3
ERR_ALIGNMENT = 4
ERR_CUDA = 5
ERR_DEVICE_TIMEOUT = 6

MLP_X_PER_TOKEN = 1
MLP_W_PER_CHANNEL = 2
MLP_PREPACKED = 4
MLP_REFERENCE_ROUNDING = 8
MLP_STATIC_SCALES = 16
MLP_WORKSPACE_KEPT = 32

_vp = ctypes.c_void_p
_i = ctypes.c_int
_i64 = ctypes.c_int64
_sz = ctypes.c_size_t
_f = ctypes.c_float

# name -> (restype, argtypes); one entry per declaration in include/i8tk.h
SIGNATURES = {
    "i8tk_status_string": (ctypes.c_char_p, [_i]),
    "i8tk_last_error": (ctypes.c_char_p, []),
    "i8tk_version": (_i, []),
    "i8tk_check_status_word": (_i, [_vp, _vp]),
    "i8tk_selftest_bounded_wait": (_i, [_vp, _i, _vp]),
    "i8tk_quantize_per_token_f32": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "i8tk_quantize_per_token_f16": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "i8tk_quantize_qkv_heads_f16": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "i8tk_dequantize_per_token_f16": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _vp]),
    "i8tk_layernorm_quantize_f16": (_i, [_vp, _vp, _vp, _i64, _i, _f, _vp]),
    "i8tk_kv_append_quantize_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "i8tk_quantize_fp16_to_int8": (_i, [_vp, _vp, _vp, _i64, _vp]),
    "i8tk_dequantize_int8_to_fp16": (_i, [_vp, _vp, _f, _i64, _vp]),
    "i8tk_decode_workspace_bytes": (_sz, [_i, _i, _i]),
    "i8tk_decode_attention_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _sz, _vp]),
    "i8tk_decode_attention_forward_q8": (_i, [_vp] * 9 + [_i] * 4 + [_vp, _sz, _vp]),
    "i8tk_decode_static_scratch_bytes": (_sz, []),
    "i8tk_decode_attention_forward_static": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "i8tk_decode_static_check_status": (_i, [_vp]),
    "i8tk_decode_attention_paged": (_i, [_vp] * 9 + [_i] * 6 + [_vp, _sz, _vp]),
    "i8tk_decode_attention_paged_checked": (_i, [_vp] * 9 + [_i] * 7 + [_vp, _sz, _vp]),
    "i8tk_decode_attention_partial": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _sz, _vp]),
    "i8tk_decode_combine_partials": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "i8tk_decode_exchange_ctas": (_i, [_i]),
    "i8tk_decode_set_exchange_spin_limit": (_i, [ctypes.c_uint]),
    "i8tk_decode_attention_seq_sharded": (_i, [_vp] * 7 + [_i, _i, _i, _vp, _sz, _vp, _vp, _i, _i,
                                               ctypes.c_uint, _vp]),
    "i8tk_decode_partial_stride": (_i, [_i]),
    "i8tk_decode_set_probe_events": (_i, [_vp, _vp]),
    "i8tk_decode_plan": (_i, [_i, _i, _i, ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "i8tk_attention_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "i8tk_attention_forward": (_i, [_vp] * 7 + [_i, _i, _i, _i, _vp, _sz, _vp]),
    "i8tk_mlp_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "i8tk_mlp_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                              _i, _i, _i, _i, _vp, _sz, _vp]),
    "i8tk_linear_i8_f16": (_i, [_vp] * 6 + [_i] * 4 + [_vp, _sz, _vp]),
    "i8tk_transpose_int8_weights": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
}

_lib = None


def load():
    """Load ``libi8tk.so`` and attach the signatures (cached)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError("%s not built: run `python build.py` in %s; there is no fallback path"
                          % (LIB_PATH, _HERE))
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError if a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error():
    return load().i8tk_last_error().decode()


def status_string(code):
    return load().i8tk_status_string(code).decode()


def check(code, what="i8tk call"):
    if code != OK:
        raise RuntimeError("%s failed: %s (%s)" % (what, status_string(code), last_error()))


def decode_plan(BH, S, head_dim):
    ns, ch = _i(0), _i(0)
    check(load().i8tk_decode_plan(BH, S, head_dim, ctypes.byref(ns), ctypes.byref(ch)), "i8tk_decode_plan")
    return ns.value, ch.value

"""The C-ABI library loads and exports every function include/i8tk.h declares
(no compute calls: runs without a GPU)."""
import os
import re

from helpers import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "i8tk.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(i8tk_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared()
    assert len(names) >= 15
    lib = cabi().load()
    for n in names:
        assert hasattr(lib, n), n
    # the ctypes table covers exactly the header
    assert sorted(cabi().SIGNATURES) == names


def test_status_strings_and_version():
    c = cabi()
    assert c.status_string(c.OK) == "ok"
    assert "workspace" in c.status_string(c.ERR_WORKSPACE)
    assert c.load().i8tk_version() >= 100
    assert c.load().i8tk_decode_partial_stride(64) == 68


def test_host_side_argument_checks_need_no_gpu():
    c = cabi()
    lib = c.load()
    assert lib.i8tk_decode_workspace_bytes(0, 16, 64) == 0
    assert lib.i8tk_decode_workspace_bytes(2, 16, 96) == 0
    assert lib.i8tk_mlp_workspace_bytes(128, 128, 256, 3) > 128 * 256 + 128 * 128 * 2   # int8 hidden + fp16 out
    assert lib.i8tk_quantize_per_token_f32(None, None, None, -1, 64, None) == c.ERR_INVALID_ARGUMENT
    assert lib.i8tk_decode_combine_partials(None, 1, 1, 64, None, None) == c.ERR_INVALID_ARGUMENT
    assert lib.i8tk_mlp_forward(None, None, None, None, None, None, None, None, None, None,
                                100, 128, 128, 0, None, 0, None) == c.ERR_INVALID_ARGUMENT

"""The reference's native launchers (C++ linkage, kernels/int8_ext.cu:27-70) as shipped in
libi8tk_compat.so: a torch-free C++ program (tests/compat_driver.cpp) links every one of them
by its C++ name, as tests/cuda/test_int8.cu:15-26 of the reference does, and compares each with
the C ABI on the same inputs.  Without a GPU only the link is checked."""
import os
import subprocess

import pytest
import torch

from helpers import pkg


def _driver():
    import importlib
    b = importlib.import_module(pkg().__name__ + ".build")
    if not os.path.exists(b.COMPAT_DRIVER) or not os.path.exists(b.COMPAT_LIB):
        b.build_lib()
        b.build_compat()
    return b.COMPAT_DRIVER


def test_driver_links_every_launcher_by_its_cpp_name():
    out = subprocess.run([_driver(), "link-only"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "linked" in out.stdout


def test_header_declares_what_the_reference_declares():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "include", "i8tk_compat.h")).read()
    for name in ("int8_attention_forward", "int8_decode_attention_forward", "int8_mlp_forward",
                 "int8_mlp_forward_per_channel", "int8_mlp_forward_per_channel_bias", "transpose_int8_weights",
                 "int8_mlp_forward_prepacked", "int8_mlp_get_output_scale", "quantize_fp16_to_int8",
                 "dequantize_int8_to_fp16"):
        assert ("void %s(" % name) in text, name


@pytest.mark.gpu
def test_launchers_match_the_c_abi_bit_for_bit():
    out = subprocess.run([_driver()], capture_output=True, text=True, timeout=300)
    print(out.stdout)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "ALL OK" in out.stdout
    assert out.stdout.count(" OK ") >= 10

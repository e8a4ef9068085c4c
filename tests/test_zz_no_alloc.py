"""The decode entry point that allocates nothing (i8tk_decode_attention_forward_static).

Some callers cannot call cudaMalloc when they need attention -- a serving
runtime's plugin hook, a process whose device memory all belongs to its own
pool -- and have no buffer to lend either.  For them the library carries a
fixed scratch block inside its own image.  This test drives that entry point
through the C ABI twice in a row (the block is shared and keeps the previous
call's contents) and checks both results against the ordinary entry point that
takes a caller-provided workspace.  Same tolerance as the other decode tests:
max-abs 2e-3 (in practice the two paths run the same kernels and agree bit for
bit).  It is collected last so a failure here cannot hide the other tests.
"""
import numpy as np
import pytest
import torch

from helpers import cabi, ext

pytestmark = pytest.mark.gpu


def _inputs(B, H, D, S, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    e = ext()
    Qi, sQ = e.quantize_per_token(torch.randn(B, H, D, device="cuda", dtype=torch.float16, generator=g))
    Ki, sK = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda", generator=g))
    Vi, sV = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda", generator=g))
    return Qi, Ki, Vi, sQ.contiguous(), sK.contiguous(), sV.contiguous()


def _call_static(lib, Qi, Ki, Vi, sQ, sK, sV):
    B, H, S, D = Ki.shape
    out = torch.empty(B, H, D, dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.i8tk_decode_attention_forward_static(Qi.data_ptr(), Ki.data_ptr(), Vi.data_ptr(), out.data_ptr(),
                                                  sQ.data_ptr(), sK.data_ptr(), sV.data_ptr(), B * H, S, D, stream)
    return rc, out


def _call_workspace(lib, Qi, Ki, Vi, sQ, sK, sV):
    B, H, S, D = Ki.shape
    out = torch.empty(B, H, D, dtype=torch.float16, device="cuda")
    wbytes = lib.i8tk_decode_workspace_bytes(B * H, S, D)
    ws = torch.empty(wbytes, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    cabi().check(lib.i8tk_decode_attention_forward(Qi.data_ptr(), Ki.data_ptr(), Vi.data_ptr(), out.data_ptr(),
                                                   sQ.data_ptr(), sK.data_ptr(), sV.data_ptr(), B * H, S, D,
                                                   ws.data_ptr(), wbytes, stream))
    return out


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    lib = cabi().load()
    assert lib.i8tk_decode_static_scratch_bytes() == 8 << 20
    first = _inputs(4, 12, 64, 3000, seed=1)          # ragged context, several splits per row
    second = _inputs(2, 8, 128, 4096, seed=2)         # other head size: the block is reused as is
    for args in (first, second, first):
        rc, got = _call_static(lib, *args)
        cabi().check(rc, "i8tk_decode_attention_forward_static")
        want = _call_workspace(lib, *args)
        torch.cuda.synchronize()
        diff = (got.float() - want.float()).abs().max().item()
        assert not torch.isnan(got).any()
        assert diff <= 2e-3, diff
    # the block's status record is reachable only through the library: no wait gave up
    assert lib.i8tk_decode_static_check_status(torch.cuda.current_stream().cuda_stream) == cabi().OK


def test_static_scratch_entry_refuses_shapes_beyond_its_block():
    lib = cabi().load()
    # many rows with a one-tile context: far more partial rows than 8 MiB holds
    BH, S, D = 200000, 64, 128
    assert lib.i8tk_decode_workspace_bytes(BH, S, D) > lib.i8tk_decode_static_scratch_bytes()
    one = torch.zeros(16, dtype=torch.int8, device="cuda")     # never dereferenced: the size check comes first
    f = torch.zeros(4, dtype=torch.float32, device="cuda")
    rc = lib.i8tk_decode_attention_forward_static(one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(),
                                                  f.data_ptr(), f.data_ptr(), f.data_ptr(), BH, S, D, None)
    assert rc == cabi().ERR_WORKSPACE
    assert "scratch" in cabi().last_error()

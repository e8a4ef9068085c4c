"""A device-side wait that runs out returns a status instead of hanging: the probe
kernel waits on a barrier nothing signals, gives up after a bounded number of
polls, records the marker, and the context stays usable."""
import pytest
import torch

from helpers import cabi, ext

pytestmark = pytest.mark.gpu


def test_wait_gives_up_and_context_survives():
    c = cabi()
    lib = c.load()
    word = torch.zeros(64, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert lib.i8tk_check_status_word(word.data_ptr(), st) == c.OK
    c.check(lib.i8tk_selftest_bounded_wait(word.data_ptr(), 2000, st))
    rc = lib.i8tk_check_status_word(word.data_ptr(), st)
    assert rc == c.ERR_DEVICE_TIMEOUT
    assert "bounded wait" in c.last_error()
    # the context is still usable
    x = torch.randn(8, 64, device="cuda")
    q, s = ext().quantize_per_token(x)
    assert torch.isfinite(s).all() and int(q.abs().max()) == 127


def test_decode_workspace_status_is_clean_after_a_normal_call():
    c = cabi()
    lib = c.load()
    e = ext()
    B, H, D, S = 2, 4, 64, 512
    Qi, sQ = e.quantize_per_token(torch.randn(B, H, D, device="cuda"))
    Ki, sK = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda"))
    Vi, sV = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda"))
    wbytes = lib.i8tk_decode_workspace_bytes(B * H, S, D)
    ws = torch.zeros(wbytes, dtype=torch.uint8, device="cuda")
    out = torch.empty(B, H, D, dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    c.check(lib.i8tk_decode_attention_forward(Qi.data_ptr(), Ki.data_ptr(), Vi.data_ptr(), out.data_ptr(),
                                              sQ.data_ptr(), sK.data_ptr(), sV.data_ptr(), B * H, S, D,
                                              ws.data_ptr(), wbytes, st))
    assert lib.i8tk_check_status_word(ws.data_ptr(), st) == c.OK

"""A device-side wait that runs out returns a status instead of hanging: the probe
kernel waits on a barrier nothing signals, gives up after a bounded number of
polls, records the marker, and the context stays usable.  The same for a real
kernel: the cross-GPU exchange of the sequence-sharded decode, run as rank 0 of a
world of two whose second rank never arrives (both "peer" buffers are local
memory, nothing faults or hangs: the wait simply runs out of its shortened
budget)."""
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


def test_exchange_kernel_gives_up_when_a_rank_never_signals():
    c = cabi()
    lib = c.load()
    e = ext()
    B, H, D, S, world = 2, 4, 64, 640, 2
    BH = B * H
    Qi, sQ = e.quantize_per_token(torch.randn(B, H, D, device="cuda"))
    Ki, sK = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda"))
    Vi, sV = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda"))
    ctas = lib.i8tk_decode_exchange_ctas(BH)
    parts = [torch.zeros(2 * world * BH * (D + 4), device="cuda") for _ in range(world)]
    flags = [torch.zeros(world * ctas, dtype=torch.int32, device="cuda") for _ in range(world)]
    pp = torch.tensor([t.data_ptr() for t in parts], dtype=torch.int64, device="cuda")
    pf = torch.tensor([t.data_ptr() for t in flags], dtype=torch.int64, device="cuda")
    wbytes = lib.i8tk_decode_workspace_bytes(BH, S, D)
    ws = torch.zeros(wbytes, dtype=torch.uint8, device="cuda")
    out = torch.empty(B, H, D, dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    c.check(lib.i8tk_decode_set_exchange_spin_limit(2000))        # a few milliseconds instead of seconds
    try:
        c.check(lib.i8tk_decode_attention_seq_sharded(
            Qi.data_ptr(), Ki.data_ptr(), Vi.data_ptr(), out.data_ptr(), sQ.data_ptr(), sK.data_ptr(), sV.data_ptr(),
            BH, S, D, ws.data_ptr(), wbytes, pp.data_ptr(), pf.data_ptr(), 0, world, 1, st))
        rc = lib.i8tk_check_status_word(ws.data_ptr(), st)
    finally:
        c.check(lib.i8tk_decode_set_exchange_spin_limit(0))
    assert rc == c.ERR_DEVICE_TIMEOUT
    words = ws[:8].view(torch.int32).cpu()
    assert int(words[1]) == ctas                                  # every CTA waited for rank 1 and gave up
    # rank 0 did publish its own rows and flags before it waited
    assert int(flags[0][:ctas].min()) == 1 and int(flags[1][:ctas].min()) == 1
    assert int(flags[0][ctas:].max()) == 0
    # the context is usable, and the next call on the same workspace starts with a clean word 0
    full = e.int8_decode_attention_forward(Qi, Ki, Vi, sQ, sK, sV)
    assert torch.isfinite(full.float()).all()
    c.check(lib.i8tk_decode_attention_forward(Qi.data_ptr(), Ki.data_ptr(), Vi.data_ptr(), out.data_ptr(),
                                              sQ.data_ptr(), sK.data_ptr(), sV.data_ptr(), BH, S, D,
                                              ws.data_ptr(), wbytes, st))
    assert lib.i8tk_check_status_word(ws.data_ptr(), st) == c.OK
    assert int(ws[:8].view(torch.int32).cpu()[1]) == ctas         # the sticky count is the caller's to reset
    assert torch.equal(out, full)


def test_ops_record_no_give_up_and_check_status_reports_clean():
    e = ext()
    x = torch.randn(1, 256, 256, device="cuda", dtype=torch.float16)
    xi, sx = e.quantize_per_token(x)
    w1 = torch.randint(-127, 128, (256, 512), dtype=torch.int8, device="cuda")
    w2 = torch.randint(-127, 128, (512, 256), dtype=torch.int8, device="cuda")
    e.int8_mlp_forward(xi, w1, w2, sx.reshape(-1), torch.full((512,), 1e-3, device="cuda"),
                       torch.full((256,), 1e-3, device="cuda"))
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        Qi, sQ = e.quantize_per_token(torch.randn(1, 4, 64, device="cuda"))
        Ki, sK = e.quantize_per_token(torch.randn(1, 4, 300, 64, device="cuda"))
        e.int8_decode_attention_forward(Qi, Ki, Ki, sQ, sK, sK)
    assert e.check_status() >= 2                                  # one scratch block per stream used

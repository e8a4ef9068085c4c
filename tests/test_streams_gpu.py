"""Calls on different streams own their workspaces and may run at the same time: results must be
those of the serial calls (the kernels of a call are chained by programmatic dependent launch,
which must not leak across streams)."""
import pytest
import torch

from helpers import ext

pytestmark = pytest.mark.gpu


def _decode_case(seed, B=4, H=8, S=3000, D=64):
    g = torch.Generator(device="cuda").manual_seed(seed)
    e = ext()
    Qi, sQ = e.quantize_per_token(torch.randn(B, H, D, device="cuda", generator=g))
    Ki, sK = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda", generator=g))
    Vi, sV = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda", generator=g))
    return [Qi, Ki, Vi, sQ.reshape(-1).contiguous(), sK.reshape(-1).contiguous(), sV.reshape(-1).contiguous()]


def test_decode_and_mlp_on_two_streams_match_serial_results():
    e = ext()
    cases = [_decode_case(s, D=64 if s % 2 else 128) for s in range(4)]
    serial = [e.int8_decode_attention_forward(*c) for c in cases]
    g = torch.Generator(device="cuda").manual_seed(11)
    M, dm, dff = 1024, 256, 1024
    xi, sx = e.quantize_per_token(torch.randn(1, M, dm, device="cuda", dtype=torch.float16, generator=g))
    w1 = torch.randint(-127, 128, (dm, dff), dtype=torch.int8, device="cuda", generator=g)
    w2 = torch.randint(-127, 128, (dff, dm), dtype=torch.int8, device="cuda", generator=g)
    s1 = torch.rand(dff, device="cuda", generator=g) * 1e-3 + 1e-3
    s2 = torch.rand(dm, device="cuda", generator=g) * 1e-3 + 1e-3
    sxf = sx.reshape(-1).contiguous()
    mlp_serial = e.int8_mlp_forward(xi, w1, w2, sxf, s1, s2)
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [[None] * len(cases) for _ in range(6)]
    mlps = []
    for rep in range(6):
        for i, c in enumerate(cases):
            with torch.cuda.stream(streams[i % 2]):
                outs[rep][i] = e.int8_decode_attention_forward(*c)
        with torch.cuda.stream(streams[rep % 2]):
            mlps.append(e.int8_mlp_forward(xi, w1, w2, sxf, s1, s2))
    torch.cuda.synchronize()
    for rep in range(6):
        for i in range(len(cases)):
            assert torch.equal(outs[rep][i], serial[i]), (rep, i)
    for o, sc in mlps:
        assert torch.equal(o, mlp_serial[0]) and torch.equal(sc, mlp_serial[1])


def test_two_large_mlp_forwards_on_two_streams():
    """Two forwards that each want nearly every SM, issued on two streams: the CTAs of the later kernels
    become resident as those of the earlier ones leave, and the CTAs that share a row block wait (bounded)
    for siblings that arrive a little later.  The results must be those of the serial calls and no wait may
    have given up."""
    e = ext()
    g = torch.Generator(device="cuda").manual_seed(21)
    shapes = [(4096, 1024, 4096), (4096, 768, 3072)]
    jobs = []
    for (M, dm, dff) in shapes:
        xi, sx = e.quantize_per_token(torch.randn(1, M, dm, device="cuda", dtype=torch.float16, generator=g))
        w1 = torch.randint(-127, 128, (dm, dff), dtype=torch.int8, device="cuda", generator=g)
        w2 = torch.randint(-127, 128, (dff, dm), dtype=torch.int8, device="cuda", generator=g)
        s1 = torch.rand(dff, device="cuda", generator=g) * 1e-4 + 1e-4
        s2 = torch.rand(dm, device="cuda", generator=g) * 1e-4 + 1e-4
        jobs.append((xi, w1, w2, sx.reshape(-1).contiguous(), s1, s2))
    serial = [e.int8_mlp_forward(*j) for j in jobs]
    torch.cuda.synchronize()
    e.check_status()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    got = [[], []]
    for rep in range(8):
        for i, j in enumerate(jobs):
            with torch.cuda.stream(streams[i]):
                got[i].append(e.int8_mlp_forward(*j))
    torch.cuda.synchronize()
    e.check_status()                                     # raises if a bounded wait ran out
    for i in range(2):
        for o, sc in got[i]:
            assert torch.equal(o, serial[i][0]) and torch.equal(sc, serial[i][1])

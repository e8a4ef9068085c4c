"""Side by side with the reference project's OWN CUDA kernels on the same GPU.

``oracle/build_ref.py`` compiles the unmodified reference kernels (its sm_80-era
mma.sync / dp4a code) for sm_100a into ``oracle/_ref/libref_kernels.so``; these
tests run both libraries on identical seeded inputs.  Skipped when that library
has not been built.  Tolerances: decode fp16 outputs within 2e-3 of each other;
MLP int8 codes within 2 steps with < 2 % mismatches (tanh.approx and
multiply-add fusion move values that sit on a rounding boundary), row scales
within 2e-3 relative.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from helpers import ext

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_kernels.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_LIB):
        pytest.skip("reference kernels not built (oracle/build_ref.py)")
    lib = ctypes.CDLL(REF_LIB)
    vp, i = ctypes.c_void_p, ctypes.c_int
    lib.ref_decode_attention_forward.argtypes = [vp] * 7 + [i] * 3
    lib.ref_mlp_forward_per_channel_bias.argtypes = [vp] * 9 + [i] * 4
    lib.ref_mlp_forward_prepacked.argtypes = [vp] * 7 + [i] * 4
    lib.ref_mlp_get_output_scale.restype = ctypes.c_float
    lib.ref_attention_forward.argtypes = [vp] * 7 + [i] * 4
    return lib


def _time(fn, iters=20, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e3      # us


def _decode_inputs(B, H, D, S, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    e = ext()
    Qi, sQ = e.quantize_per_token(torch.randn(B, H, D, device="cuda", dtype=torch.float16, generator=g))
    Ki, sK = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda", generator=g))
    Vi, sV = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda", generator=g))
    return Qi, Ki, Vi, sQ.contiguous(), sK.contiguous(), sV.contiguous()


@pytest.mark.parametrize("B,H,D,S", [(2, 4, 64, 1000), (2, 4, 128, 4096), (1, 1, 64, 33), (8, 12, 64, 8192),
                                     (4, 8, 128, 8192)])
def test_decode_matches_reference_kernel(ref, B, H, D, S):
    Qi, Ki, Vi, sQ, sK, sV = _decode_inputs(B, H, D, S, seed=S + D)
    ours = ext().int8_decode_attention_forward(Qi, Ki, Vi, sQ, sK, sV)
    theirs = torch.empty_like(ours)
    rc = ref.ref_decode_attention_forward(Qi.data_ptr(), Ki.data_ptr(), Vi.data_ptr(), theirs.data_ptr(),
                                          sQ.data_ptr(), sK.data_ptr(), sV.data_ptr(), B * H, S, D)
    torch.cuda.synchronize()
    assert rc == 0
    assert (ours.float() - theirs.float()).abs().max().item() < 2e-3


def test_decode_speed_beside_reference_kernel(ref, capsys):
    """Serving-scale shapes: the new kernels must not be slower than the reference's own
    kernels recompiled for this GPU (they are several times faster; the factor is printed)."""
    lines = []
    for (B, H, D, S) in [(32, 12, 64, 8192), (16, 32, 128, 8192)]:
        Qi, Ki, Vi, sQ, sK, sV = _decode_inputs(B, H, D, S, seed=1)
        out = torch.empty(B, H, D, dtype=torch.float16, device="cuda")
        t_ours = _time(lambda: ext().int8_decode_attention_forward(Qi, Ki, Vi, sQ, sK, sV))
        t_ref = _time(lambda: ref.ref_decode_attention_forward(Qi.data_ptr(), Ki.data_ptr(), Vi.data_ptr(),
                                                               out.data_ptr(), sQ.data_ptr(), sK.data_ptr(),
                                                               sV.data_ptr(), B * H, S, D))
        gb = 2 * B * H * S * D / 1e3
        lines.append(f"decode B{B} H{H} D{D} ctx{S}: ours {t_ours:.1f} us ({gb / t_ours:.0f} GB/s), "
                     f"reference kernel {t_ref:.1f} us ({gb / t_ref:.0f} GB/s), x{t_ref / t_ours:.2f}")
        assert t_ours < t_ref
    with capsys.disabled():
        print("\n" + "\n".join(lines))


def _mlp_inputs(M, dm, dff, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    e = ext()
    xi, sx = e.quantize_per_token(torch.randn(1, M, dm, device="cuda", dtype=torch.float16, generator=g))
    W1 = torch.randn(dm, dff, device="cuda", generator=g) * 0.02
    W2 = torch.randn(dff, dm, device="cuda", generator=g) * 0.02
    s1 = (W1.abs().amax(dim=0).clamp(min=1e-8) / 127.0).contiguous()
    s2 = (W2.abs().amax(dim=0).clamp(min=1e-8) / 127.0).contiguous()
    w1i = (W1 / s1).round().clamp(-128, 127).to(torch.int8).contiguous()
    w2i = (W2 / s2).round().clamp(-128, 127).to(torch.int8).contiguous()
    b1 = (torch.randn(dff, device="cuda", generator=g) * 0.01).contiguous()
    return xi, w1i, w2i, sx.reshape(-1).contiguous(), s1, s2, b1


@pytest.mark.parametrize("M,dm,dff", [(256, 256, 512), (512, 768, 3072), (1024, 1024, 4096)])
def test_mlp_matches_reference_kernel(ref, M, dm, dff):
    xi, w1i, w2i, sx, s1, s2, b1 = _mlp_inputs(M, dm, dff, seed=M)
    ours, ours_sc = ext().int8_mlp_forward_per_channel_bias(xi, w1i, w2i, sx, s1, s2, b1)
    theirs = torch.empty_like(ours)
    theirs_sc = torch.empty(M, device="cuda")
    rc = ref.ref_mlp_forward_per_channel_bias(xi.data_ptr(), w1i.data_ptr(), w2i.data_ptr(), theirs.data_ptr(),
                                              sx.data_ptr(), s1.data_ptr(), s2.data_ptr(), b1.data_ptr(),
                                              theirs_sc.data_ptr(), 1, M, dm, dff)
    torch.cuda.synchronize()
    assert rc == 0
    d = (ours.int() - theirs.int()).abs()
    assert int(d.max()) <= 2
    assert float((d != 0).float().mean()) < 0.02
    assert torch.allclose(ours_sc, theirs_sc, rtol=2e-3, atol=1e-9)


def test_mlp_speed_beside_reference_kernel(ref, capsys):
    M, dm, dff = 4096, 1024, 4096
    xi, w1i, w2i, sx, s1, s2, b1 = _mlp_inputs(M, dm, dff, seed=3)
    out = torch.empty_like(xi)
    sc = torch.empty(M, device="cuda")
    t_ours = _time(lambda: ext().int8_mlp_forward_per_channel_bias(xi, w1i, w2i, sx, s1, s2, b1))
    t_ref = _time(lambda: ref.ref_mlp_forward_per_channel_bias(xi.data_ptr(), w1i.data_ptr(), w2i.data_ptr(),
                                                               out.data_ptr(), sx.data_ptr(), s1.data_ptr(),
                                                               s2.data_ptr(), b1.data_ptr(), sc.data_ptr(),
                                                               1, M, dm, dff))
    tops = 4.0 * M * dm * dff / 1e6
    with capsys.disabled():
        print(f"\nMLP M{M} {dm}->{dff}: ours {t_ours:.1f} us ({tops / t_ours:.0f} TOPS), reference kernel "
              f"{t_ref:.1f} us ({tops / t_ref:.0f} TOPS), x{t_ref / t_ours:.2f}")
    assert t_ours < t_ref


def test_prefill_speed_beside_reference_kernel(ref, capsys):
    lines = []
    for (B, H, S, D) in [(8, 8, 4096, 64), (4, 8, 4096, 128)]:
        g = torch.Generator(device="cuda").manual_seed(2)
        e = ext()
        t = []
        for _ in range(3):
            xi, sx = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda", dtype=torch.float16, generator=g))
            t.append((xi, sx.reshape(-1).contiguous()))
        (Qi, sQ), (Ki, sK), (Vi, sV) = t
        out = torch.empty(B, H, S, D, dtype=torch.float16, device="cuda")
        t_ours = _time(lambda: e.int8_attention_forward(Qi, Ki, Vi, sQ, sK, sV), iters=10)
        t_ref = _time(lambda: ref.ref_attention_forward(Qi.data_ptr(), Ki.data_ptr(), Vi.data_ptr(), out.data_ptr(),
                                                        sQ.data_ptr(), sK.data_ptr(), sV.data_ptr(), B, H, S, D),
                      iters=10)
        tops = 4.0 * B * H * S * S * D / 1e6
        lines.append(f"prefill B{B} H{H} S{S} D{D}: ours {t_ours:.0f} us ({tops / t_ours:.0f} TOPS), "
                     f"reference kernel {t_ref:.0f} us ({tops / t_ref:.0f} TOPS), x{t_ref / t_ours:.2f}")
        assert t_ours < t_ref
    with capsys.disabled():
        print("\n" + "\n".join(lines))

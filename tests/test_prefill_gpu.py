"""INT8 prefill attention: CUDA path (tcgen05 QK^T and PV) vs the oracle.

The reference accepts max-abs 0.1 against its fp16 baseline on the dequantised
operands (tests/test_int8.py:99-127, common/correctness.py:23).  P*sV and V pass
through fp16 here exactly as there, so the bar used is tighter: max-abs 2e-2 and
cosine > 0.9999 against a float64 evaluation of the same dequantised attention."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import decode as odec, quant
from helpers import ext, cabi, cosine

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_kernels.so")


def _case(B, H, S, D, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    mk = lambda: (rng.standard_normal((B, H, S, D)) * scale).astype(np.float16)
    out = []
    for x in (mk(), mk(), mk()):
        out.extend(quant.quantize_per_token(x))
    Qi, sQ, Ki, sK, Vi, sV = out
    return Qi, Ki, Vi, sQ, sK, sV


def _run(args):
    t = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in args]
    o = ext().int8_attention_forward(*t)
    assert o.dtype == torch.float16 and tuple(o.shape) == args[0].shape
    return o.float().cpu().numpy()


@pytest.mark.parametrize("B,H,S,D", [(1, 1, 128, 64), (1, 1, 128, 128), (2, 3, 256, 64), (2, 3, 384, 128),
                                     (2, 8, 512, 64), (2, 8, 512, 128), (1, 4, 1024, 128), (1, 2, 2048, 64),
                                     (1, 2, 640, 64), (1, 1, 896, 128),
                                     # ragged lengths (the reference's scalar-fallback shapes): partial last tile
                                     (1, 1, 1, 64), (2, 2, 63, 128), (1, 3, 129, 64), (2, 2, 200, 128),
                                     (1, 2, 1000, 64), (1, 1, 2049, 128),
                                     # head_dim 256 (kernels/int8_attention.cu:1012, tests/test_int8.py:82-85): 64-position tiles
                                     (1, 1, 128, 256), (2, 2, 256, 256), (1, 3, 512, 256), (1, 2, 1024, 256),
                                     (1, 1, 1, 256), (2, 2, 63, 256), (1, 2, 200, 256), (1, 1, 1090, 256)])
def test_vs_oracle(B, H, S, D):
    args = _case(B, H, S, D, seed=S + D)
    out = _run(args)
    ref = odec.prefill_attention(*args)
    assert not np.isnan(out).any()
    assert np.abs(out - ref).max() < 2e-2, np.abs(out - ref).max()
    assert cosine(out, ref) > 0.9999


def test_peaky_scores_exercise_the_lazy_maximum():
    # large-magnitude q/k: scores span hundreds of log2 units, the running maximum moves often
    args = _case(1, 2, 512, 64, seed=7, scale=4.0)
    out = _run(args)
    ref = odec.prefill_attention(*args)
    assert np.abs(out - ref).max() < 5e-2
    assert cosine(out, ref) > 0.999


def test_degenerate_inputs():
    B, H, S, D = 1, 2, 256, 128
    z = np.zeros((B, H, S, D), np.float32)
    Zi, sZ = quant.quantize_per_token(z)
    out = _run((Zi, Zi, Zi, sZ, sZ, sZ))
    assert np.all(out == 0.0)
    o = np.ones((B, H, S, D), np.float32)
    Oi, sO = quant.quantize_per_token(o)
    out = _run((Oi, Oi, Oi, sO, sO, sO))
    assert np.allclose(out, 1.0, atol=2e-3)


def test_unsupported_shapes_raise():
    e = ext()
    mk = lambda S, D: torch.zeros(1, 1, S, D, dtype=torch.int8, device="cuda")
    sc = lambda S: torch.ones(S, device="cuda")
    with pytest.raises(RuntimeError, match="head_dim 64, 128 or 256"):
        e.int8_attention_forward(mk(128, 96), mk(128, 96), mk(128, 96), sc(128), sc(128), sc(128))
    with pytest.raises(RuntimeError, match="shape mismatch"):
        e.int8_attention_forward(mk(128, 64), mk(256, 64), mk(128, 64), sc(128), sc(128), sc(128))


def test_matches_reference_kernel_when_built():
    if not os.path.exists(REF_LIB):
        pytest.skip("reference kernels not built (oracle/build_ref.py)")
    ref = ctypes.CDLL(REF_LIB)
    ref.ref_attention_forward.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 4
    for (B, H, S, D) in [(2, 4, 512, 64), (2, 4, 512, 128), (1, 4, 512, 256)]:
        args = _case(B, H, S, D, seed=11)
        t = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in args]
        ours = ext().int8_attention_forward(*t)
        theirs = torch.empty_like(ours)
        rc = ref.ref_attention_forward(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), theirs.data_ptr(),
                                       t[3].data_ptr(), t[4].data_ptr(), t[5].data_ptr(), B, H, S, D)
        torch.cuda.synchronize()
        assert rc == 0
        assert (ours.float() - theirs.float()).abs().max().item() < 2e-2

"""Per-token quantiser: CUDA kernel vs the oracle and the golden vectors (bit-exact)."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import quant
from helpers import ext, cabi, gold

pytestmark = pytest.mark.gpu


def _check(x_np):
    x = torch.from_numpy(np.ascontiguousarray(x_np)).cuda()
    q, s = ext().quantize_per_token(x)
    q_ref, s_ref = quant.quantize_per_token(x_np)
    assert q.dtype == torch.int8 and s.dtype == torch.float32
    assert tuple(q.shape) == x_np.shape and tuple(s.shape) == x_np.shape[:-1]
    assert np.array_equal(q.cpu().numpy(), q_ref)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))


def test_golden_vectors_bit_exact():
    g = gold("quantize_per_token.npz")
    names = sorted(k[:-3] for k in g.files if k.endswith("__x"))
    for n in names:
        x = torch.from_numpy(g[n + "__x"]).cuda()
        q, s = ext().quantize_per_token(x)
        assert np.array_equal(q.cpu().numpy(), g[n + "__q"]), n
        assert np.array_equal(s.cpu().numpy().view(np.uint32), g[n + "__s"].view(np.uint32)), n


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("shape", [
    (1, 64), (5, 64), (1, 12, 1024, 64), (3, 7, 33, 128), (4096, 768), (512, 1024),
    (257, 3072), (100, 4096), (9, 37), (3, 1), (1000, 8), (17, 96), (33, 2048), (5, 8192)])
def test_matches_oracle(dtype, shape):
    rng = np.random.default_rng(hash(shape) % (2 ** 31))
    x = rng.standard_normal(shape).astype(dtype)
    _check(x)


def test_edge_rows():
    x = np.zeros((8, 128), dtype=np.float32)
    x[1] = 1.0
    x[2] = -3.5
    x[3, 5] = 1e30
    x[4] = 1e-20
    x[5] = np.linspace(-1, 1, 128)
    x[6, ::2] = 0.5
    x[6, 0] = 127.0            # scale 1 -> exact .5 ties
    x[7, 3] = -1e-9
    _check(x)
    x[3, 5] = 6.0e4            # largest magnitude that stays finite in fp16
    _check(x.astype(np.float16))


def test_outlier_channels_distribution():
    # 1% of channels scaled x20 (the outlier-column construction of the serving configs)
    rng = np.random.default_rng(7)
    x = rng.standard_normal((64, 333, 128)).astype(np.float32)
    x[..., 17] *= 20.0
    _check(x)


def test_empty_and_errors():
    lib = cabi().load()
    x = torch.empty(0, 64, device="cuda")
    q, s = ext().quantize_per_token(x)
    assert q.numel() == 0 and s.numel() == 0
    with pytest.raises(RuntimeError):
        ext().quantize_per_token(torch.zeros(4, 64, device="cuda", dtype=torch.float64))
    with pytest.raises(RuntimeError):
        ext().quantize_per_token(torch.zeros(4, 64))
    assert lib.i8tk_quantize_per_token_f32(None, None, None, 4, 64, None) == cabi().ERR_INVALID_ARGUMENT
    assert "null" in cabi().last_error()


def test_large_rows_property():
    """Full-size property check: codes in range, |x - q*s| <= s/2, absmax row -> +-127."""
    torch.manual_seed(0)
    x = torch.randn(32 * 12 * 4096, 64, device="cuda")
    q, s = ext().quantize_per_token(x)
    err = (x - q.float() * s[:, None]).abs()
    assert bool((err <= s[:, None] * 0.5001).all())      # half a step, plus fp32 rounding of x/s
    assert int(q.abs().amax(dim=1).min()) == 127
    # scales bit-exact against the CPU torch arithmetic on a slice (CUDA torch turns
    # `t / 127.0` into a multiply by the rounded reciprocal, which is 1 ulp off in
    # some rows, so the device-side torch result is not the yardstick)
    xs = x[:200000].cpu()
    ref_s = xs.abs().amax(dim=1).clamp(min=1e-8) / 127.0
    assert torch.equal(s[:200000].cpu(), ref_s)
    ref_q = (xs / ref_s[:, None]).round().clamp(-128, 127).to(torch.int8)
    assert torch.equal(q[:200000].cpu(), ref_q)


def test_per_tensor_roundtrip():
    lib = cabi().load()
    x = torch.randn(10000, device="cuda").half()
    q = torch.empty(10000, device="cuda", dtype=torch.int8)
    sc = torch.zeros(1, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    cabi().check(lib.i8tk_quantize_fp16_to_int8(x.data_ptr(), q.data_ptr(), sc.data_ptr(), 10000, st))
    q_ref, s_ref = quant.quantize_per_tensor(x.cpu().numpy())
    assert np.float32(sc.item()) == s_ref
    assert np.array_equal(q.cpu().numpy(), q_ref)
    out = torch.empty(10000, device="cuda", dtype=torch.float16)
    cabi().check(lib.i8tk_dequantize_int8_to_fp16(q.data_ptr(), out.data_ptr(),
                                                  ctypes.c_float(float(s_ref)), 10000, st))
    assert torch.equal(out.cpu(), (q.cpu().float() * float(s_ref)).half())

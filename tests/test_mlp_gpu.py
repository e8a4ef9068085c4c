"""Fused INT8 MLP: CUDA path (tcgen05 GEMMs) vs the oracle.

Tolerances: against the reference's dequantised simulation (sim_mlp) the
reference itself accepts max-abs 0.05 (validation/validate_int8.py:54); the
benchmark target is cosine >= 0.9999.  Against the stage-by-stage restatement of
the reference kernel (oracle.mlp.kernel_mlp) int8 codes may differ by one step
where a value sits on a rounding boundary (the GPU uses exp2-based GELU and
fused multiply-adds), so the mismatch RATE and the size of a mismatch are bounded.
"""
import numpy as np
import pytest
import torch

from oracle import mlp as omlp, quant
from helpers import ext, cabi, gold, cosine

pytestmark = pytest.mark.gpu


def _prep(x, W1, W2):
    T, dm = x.shape[-2], x.shape[-1]
    xi, sx = quant.quantize_per_token(x.reshape(T, dm))
    w1i, s1 = quant.quantize_per_channel_w(W1)
    w2i, s2 = quant.quantize_per_channel_w(W2)
    return xi, w1i, w2i, sx, s1, s2


def _cuda(*arrs):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrs]


def _run_pc(xi, w1i, w2i, sx, s1, s2, b1=None):
    T, dm = xi.shape
    x_t, sx_t, w1_t, s1_t, w2_t, s2_t = _cuda(xi.reshape(1, T, dm), sx, w1i, s1, w2i, s2)
    if b1 is None:
        out, osc = ext().int8_mlp_forward(x_t, w1_t, w2_t, sx_t, s1_t, s2_t)
    else:
        out, osc = ext().int8_mlp_forward_per_channel_bias(x_t, w1_t, w2_t, sx_t, s1_t, s2_t, _cuda(b1)[0])
    assert out.dtype == torch.int8 and tuple(out.shape) == (1, T, dm)
    assert osc.dtype == torch.float32 and tuple(osc.shape) == (T,)
    return out.cpu().numpy().reshape(T, dm), osc.cpu().numpy()


def _compare_with_kernel_oracle(out_i8, out_sc, ref, max_rate=0.02, scale_rtol=2e-3):
    mism = out_i8.astype(np.int32) - ref["out_i8"].astype(np.int32)
    rate = float((mism != 0).mean())
    assert np.abs(mism).max() <= 2, np.abs(mism).max()
    assert rate < max_rate, rate
    assert np.allclose(out_sc, ref["out_scale"], rtol=scale_rtol, atol=1e-9)
    return rate


def test_golden_simulation_tile_case():
    g = gold("mlp_sim.npz")
    x, W1, W2 = g["tile__x"], g["tile__W1"], g["tile__W2"]
    args = _prep(x, W1, W2)
    out_i8, out_sc = _run_pc(*args)
    deq = out_i8.astype(np.float32) * out_sc[:, None]
    ref = g["tile__out"]
    assert np.abs(deq - ref).max() < 0.05
    assert cosine(deq, ref) > 0.9999
    _compare_with_kernel_oracle(out_i8, out_sc, omlp.kernel_mlp(*args))


@pytest.mark.parametrize("T,dm,dff,bias", [(128, 128, 128, False), (256, 256, 512, True), (512, 768, 3072, True),
                                           (256, 1024, 4096, False), (384, 384, 640, True), (1024, 128, 256, False)])
def test_shapes_vs_oracle(T, dm, dff, bias):
    rng = np.random.default_rng(T + dm + dff)
    x = rng.standard_normal((T, dm)).astype(np.float16)
    W1 = (rng.standard_normal((dm, dff)) * 0.02).astype(np.float32)
    W2 = (rng.standard_normal((dff, dm)) * 0.02).astype(np.float32)
    b1 = (rng.standard_normal(dff) * 0.01).astype(np.float32) if bias else None
    args = _prep(x, W1, W2)
    out_i8, out_sc = _run_pc(*args, b1=b1)
    ref = omlp.kernel_mlp(*args, b1=b1)
    _compare_with_kernel_oracle(out_i8, out_sc, ref)
    deq = out_i8.astype(np.float32) * out_sc[:, None]
    sim = omlp.sim_mlp(x, W1, W2, b1=b1)["out"]
    assert cosine(deq, sim) > 0.9999
    assert np.abs(deq - sim).max() < 0.05


def test_edge_datasets_zeros_constant_outlier():
    T, dm, dff = 128, 256, 512
    # zeros: every stage is zero, scales hit the 1e-8 clamp
    z = np.zeros((T, dm), np.float32)
    args = _prep(z, np.zeros((dm, dff), np.float32), np.zeros((dff, dm), np.float32))
    out_i8, out_sc = _run_pc(*args)
    assert np.all(out_i8 == 0)
    assert np.allclose(out_sc, 1e-8 / 127.0)
    # constant inputs: single-code quantisation must be exact
    args = _prep(np.ones((T, dm), np.float32), np.full((dm, dff), 0.01, np.float32),
                 np.full((dff, dm), 0.01, np.float32))
    out_i8, out_sc = _run_pc(*args)
    ref = omlp.kernel_mlp(*args)
    assert np.array_equal(out_i8, ref["out_i8"])
    assert np.allclose(out_sc, ref["out_scale"], rtol=1e-4)
    # outlier channels in x (1% of channels x 20)
    rng = np.random.default_rng(3)
    x = rng.standard_normal((T, dm)).astype(np.float32)
    x[:, rng.permutation(dm)[:3]] *= 20.0
    W1 = (rng.standard_normal((dm, dff)) * 0.02).astype(np.float32)
    W2 = (rng.standard_normal((dff, dm)) * 0.02).astype(np.float32)
    args = _prep(x, W1, W2)
    out_i8, out_sc = _run_pc(*args)
    _compare_with_kernel_oracle(out_i8, out_sc, omlp.kernel_mlp(*args))


def test_scalar_overload_and_prepacked():
    rng = np.random.default_rng(9)
    T, dm, dff = 256, 256, 512
    x = rng.standard_normal((T, dm)).astype(np.float16)
    W1 = (rng.standard_normal((dm, dff)) * 0.02).astype(np.float16)
    W2 = (rng.standard_normal((dff, dm)) * 0.02).astype(np.float16)
    xi, sx = quant.quantize_per_tensor(x)
    w1i, s1 = quant.quantize_per_tensor(W1)
    w2i, s2 = quant.quantize_per_tensor(W2)
    x_t, w1_t, w2_t = _cuda(xi.reshape(2, T // 2, dm), w1i, w2i)
    out, osc = ext().int8_mlp_forward(x_t, w1_t, w2_t, float(sx), float(s1), float(s2))
    assert isinstance(osc, float) and tuple(out.shape) == (2, T // 2, dm)
    ref = omlp.kernel_mlp(xi, w1i, w2i, sx, s1, s2, per_token_out=False)
    o = out.cpu().numpy().reshape(T, dm)
    mism = o.astype(np.int32) - ref["out_i8"].astype(np.int32)
    assert np.abs(mism).max() <= 2 and float((mism != 0).mean()) < 0.02
    assert abs(osc - float(ref["out_scale"])) <= 2e-3 * float(ref["out_scale"])
    # against the fp16 baseline on dequantised operands, atol 0.1 (tests/test_int8.py:129-154)
    xd = xi.astype(np.float32) * sx
    base = omlp.gelu_tanh(xd @ (w1i.astype(np.float32) * s1)) @ (w2i.astype(np.float32) * s2)
    assert np.abs(o.astype(np.float32) * osc - base).max() < 0.1
    # prepacked == non-prepacked, bit for bit
    W1T, W2T = ext().transpose_int8_weights(w1_t, w2_t)
    assert torch.equal(W1T, w1_t.t().contiguous()) and torch.equal(W2T, w2_t.t().contiguous())
    out2, osc2 = ext().int8_mlp_forward_prepacked(x_t, W1T, W2T, float(sx), float(s1), float(s2))
    assert torch.equal(out, out2) and osc == osc2


def test_length_one_scale_tensors_broadcast():
    rng = np.random.default_rng(1)
    T, dm, dff = 128, 128, 256
    x = rng.standard_normal((T, dm)).astype(np.float16)
    W1 = (rng.standard_normal((dm, dff)) * 0.02).astype(np.float16)
    W2 = (rng.standard_normal((dff, dm)) * 0.02).astype(np.float16)
    xi, sx = quant.quantize_per_tensor(x)
    w1i, s1 = quant.quantize_per_tensor(W1)
    w2i, s2 = quant.quantize_per_tensor(W2)
    x_t, w1_t, w2_t = _cuda(xi.reshape(1, T, dm), w1i, w2i)
    one = lambda v: torch.full((1,), float(v), device="cuda")
    out, osc = ext().int8_mlp_forward(x_t, w1_t, w2_t, one(sx), one(s1), one(s2))
    ref = omlp.kernel_mlp(xi, w1i, w2i, sx, s1, s2, per_token_out=True)
    _compare_with_kernel_oracle(out.cpu().numpy().reshape(T, dm), osc.cpu().numpy(), ref)


def test_transpose_odd_shapes():
    for r, c in [(128, 256), (100, 36), (7, 5), (64, 64), (130, 258)]:
        a = torch.randint(-128, 128, (r, c), dtype=torch.int8, device="cuda")
        b = torch.randint(-128, 128, (c, r), dtype=torch.int8, device="cuda")
        at, bt = ext().transpose_int8_weights(a, b)
        assert torch.equal(at, a.t().contiguous()) and torch.equal(bt, b.t().contiguous())


def test_argument_errors():
    e = ext()
    x = torch.zeros(1, 128, 128, dtype=torch.int8, device="cuda")
    W1 = torch.zeros(128, 256, dtype=torch.int8, device="cuda")
    W2 = torch.zeros(256, 128, dtype=torch.int8, device="cuda")
    s = lambda n: torch.ones(n, device="cuda")
    with pytest.raises(RuntimeError, match="W1 shape mismatch"):
        e.int8_mlp_forward(x, W2, W2, s(128), s(256), s(128))
    with pytest.raises(RuntimeError, match="scale_x must have"):
        e.int8_mlp_forward(x, W1, W2, s(5), s(256), s(128))
    with pytest.raises(RuntimeError, match="bias1 must have d_ff"):
        e.int8_mlp_forward_per_channel_bias(x, W1, W2, s(128), s(256), s(128), s(3))
    with pytest.raises(RuntimeError, match="must be int8"):
        e.int8_mlp_forward(x.float(), W1, W2, s(128), s(256), s(128))
    with pytest.raises(RuntimeError, match="static-scale mode"):      # static scales are per tensor, one output scale
        lib0 = cabi().load()
        ws0 = torch.empty(lib0.i8tk_mlp_workspace_bytes(128, 128, 256, 16 | 1), dtype=torch.uint8, device="cuda")
        cabi().check(lib0.i8tk_mlp_forward(x.data_ptr(), W1.data_ptr(), W2.data_ptr(), x.data_ptr(), s(128).data_ptr(),
                                           s(256).data_ptr(), s(128).data_ptr(), None, None, s(1).data_ptr(), 128, 128,
                                           256, 16 | 1, ws0.data_ptr(), ws0.numel(), None))
    with pytest.raises(RuntimeError, match="tile multiples"):
        e.int8_mlp_forward_prepacked(torch.zeros(1, 4, 128, dtype=torch.int8, device="cuda"),
                                     W1.t().contiguous(), W2.t().contiguous(), 1.0, 1.0, 1.0)
    lib = cabi().load()
    assert lib.i8tk_mlp_forward(None, None, None, None, None, None, None, None, None, None,
                                128, 128, 128, 0, None, 0, None) == cabi().ERR_INVALID_ARGUMENT
    ws = torch.empty(256, dtype=torch.uint8, device="cuda")
    o = torch.empty_like(x)
    sc = s(256)
    rc = lib.i8tk_mlp_forward(x.data_ptr(), W1.data_ptr(), W2.data_ptr(), o.data_ptr(), sc.data_ptr(),
                              sc.data_ptr(), sc.data_ptr(), None, sc.data_ptr(), None, 128, 128, 256, 3,
                              ws.data_ptr(), 256, None)
    assert rc == cabi().ERR_WORKSPACE


@pytest.mark.parametrize("T", [1, 7, 100, 129, 300, 1000])
def test_any_number_of_rows(T):
    """Row counts that are not multiples of the 128-row tile (the reference takes its static-scale
    fallback there, kernels/int8_mlp.cu:1023-1026): same results as the rows inside a padded batch."""
    torch.manual_seed(T)
    e = ext()
    dm, dff = 256, 512
    Tp = ((T + 127) // 128) * 128
    x = torch.randn(1, Tp, dm, device="cuda", dtype=torch.float16)
    xi, sx = e.quantize_per_token(x)
    w1i, s1 = quant.quantize_per_channel_w((torch.randn(dm, dff) * 0.05).numpy())
    w2i, s2 = quant.quantize_per_channel_w((torch.randn(dff, dm) * 0.05).numpy())
    w1_t, s1_t, w2_t, s2_t = _cuda(w1i, s1, w2i, s2)
    b1 = torch.randn(dff, device="cuda") * 0.01
    sxf = sx.reshape(-1).contiguous()
    full, full_sc = e.int8_mlp_forward_per_channel_bias(xi, w1_t, w2_t, sxf, s1_t, s2_t, b1)
    part, part_sc = e.int8_mlp_forward_per_channel_bias(xi[:, :T].contiguous(), w1_t, w2_t, sxf[:T].contiguous(),
                                                        s1_t, s2_t, b1)
    assert part.shape == (1, T, dm) and part_sc.shape == (T,)
    assert torch.equal(part[0], full[0, :T]) and torch.equal(part_sc, full_sc[:T])
    # legacy per-tensor surface on the same rows
    o, sc = e.int8_mlp_forward(xi[:, :T].contiguous(), w1_t, w2_t, 0.02, 0.001, 0.001)
    assert o.shape == (1, T, dm) and sc > 0


@pytest.mark.parametrize("M,dm,dff", [(4096, 768, 3072),     # benchmark geometry: 3 tiles per CTA in GEMM1
                                      (16384, 1024, 4096),   # 15 tiles per CTA, 16 tiles per row block
                                      (1024, 256, 8192),     # 32 tiles per row block: maxima not read ahead
                                      (4900, 1024, 1024)])   # GEMM2 on CTA pairs, 39 row blocks: one CTA of the last pair has no rows
def test_full_size_config_properties(M, dm, dff):
    """Large geometries (several tiles per persistent CTA, requantisation deferred by a tile):
    determinism, row independence (a row's result does not depend on the other rows) and the
    oracle on sampled rows."""
    torch.manual_seed(0)
    e = ext()
    x = torch.randn(1, M, dm, device="cuda", dtype=torch.float16)
    W1 = torch.randn(dm, dff, device="cuda") * 0.02
    W2 = torch.randn(dff, dm, device="cuda") * 0.02
    b1 = torch.randn(dff, device="cuda") * 0.01
    xi, sx = e.quantize_per_token(x)
    w1i, s1 = quant.quantize_per_channel_w(W1.cpu().numpy())
    w2i, s2 = quant.quantize_per_channel_w(W2.cpu().numpy())
    w1_t, s1_t, w2_t, s2_t = _cuda(w1i, s1, w2i, s2)
    out, osc = e.int8_mlp_forward_per_channel_bias(xi, w1_t, w2_t, sx.reshape(-1), s1_t, s2_t, b1)
    out_b, osc_b = e.int8_mlp_forward_per_channel_bias(xi, w1_t, w2_t, sx.reshape(-1), s1_t, s2_t, b1)
    assert torch.equal(out, out_b) and torch.equal(osc, osc_b)
    sub = slice(M // 2, M // 2 + 128)
    out_s, osc_s = e.int8_mlp_forward_per_channel_bias(xi[:, sub].contiguous(), w1_t, w2_t,
                                                       sx.reshape(-1)[sub].contiguous(), s1_t, s2_t, b1)
    assert torch.equal(out_s[0], out[0, sub]) and torch.equal(osc_s, osc[sub])
    last = slice(M - (M % 128 or 128), M)                       # the last, possibly partial, row block
    out_l, osc_l = e.int8_mlp_forward_per_channel_bias(xi[:, last].contiguous(), w1_t, w2_t,
                                                       sx.reshape(-1)[last].contiguous(), s1_t, s2_t, b1)
    assert torch.equal(out_l[0], out[0, last]) and torch.equal(osc_l, osc[last])
    e.check_status()                                            # raises if any bounded wait ran out
    # prepacked weights ([N][K], K-major operand descriptors) through the C ABI: the same bytes
    c = cabi()
    lib = c.load()
    W1T, W2T = e.transpose_int8_weights(w1_t, w2_t)
    flags = c.MLP_X_PER_TOKEN | c.MLP_W_PER_CHANNEL | c.MLP_PREPACKED
    wb = lib.i8tk_mlp_workspace_bytes(M, dm, dff, flags)
    ws = torch.empty(wb, dtype=torch.uint8, device="cuda")
    out_p = torch.empty_like(out)
    osc_p = torch.empty_like(osc)
    c.check(lib.i8tk_mlp_forward(xi.data_ptr(), W1T.data_ptr(), W2T.data_ptr(), out_p.data_ptr(),
                                 sx.reshape(-1).data_ptr(), s1_t.data_ptr(), s2_t.data_ptr(), b1.data_ptr(),
                                 osc_p.data_ptr(), None, M, dm, dff, flags, ws.data_ptr(), wb,
                                 torch.cuda.current_stream().cuda_stream))
    assert lib.i8tk_check_status_word(ws.data_ptr(), torch.cuda.current_stream().cuda_stream) == c.OK
    assert torch.equal(out_p, out) and torch.equal(osc_p, osc)
    ref = omlp.kernel_mlp(xi[0, sub].cpu().numpy(), w1i, w2i, sx.reshape(-1)[sub].cpu().numpy(), s1, s2,
                          b1=b1.cpu().numpy())
    _compare_with_kernel_oracle(out_s[0].cpu().numpy(), osc_s.cpu().numpy(), ref)


def test_reference_rounding_mode_matches_the_stage_by_stage_restatement():
    """With I8TK_MLP_REFERENCE_ROUNDING the first epilogue follows the reference's source operation by
    operation (kernels/int8_mlp.cu:437-440, kernels/int8_common.cuh:9-13), so what is left against
    oracle.mlp.kernel_mlp is tanhf against numpy's tanh (an ulp now and then): at least ten times
    fewer differing codes than the default build, and none off by more than one step."""
    rng = np.random.default_rng(77)
    T, dm, dff = 512, 768, 3072
    x = rng.standard_normal((T, dm)).astype(np.float16)
    W1 = (rng.standard_normal((dm, dff)) * 0.02).astype(np.float32)
    W2 = (rng.standard_normal((dff, dm)) * 0.02).astype(np.float32)
    b1 = (rng.standard_normal(dff) * 0.01).astype(np.float32)
    args = _prep(x, W1, W2)
    ref = omlp.kernel_mlp(*args, b1=b1)
    fast_i8, fast_sc = _run_pc(*args, b1=b1)
    was = ext().set_mlp_reference_rounding(True)
    try:
        exact_i8, exact_sc = _run_pc(*args, b1=b1)
    finally:
        ext().set_mlp_reference_rounding(was)
    rate_fast = float((fast_i8 != ref["out_i8"]).mean())
    rate_exact = float((exact_i8 != ref["out_i8"]).mean())
    print(f"int8 output codes differing from the restatement: default {100 * rate_fast:.3f} %, "
          f"reference rounding {100 * rate_exact:.4f} %")
    assert np.abs(exact_i8.astype(np.int32) - ref["out_i8"].astype(np.int32)).max() <= 1
    assert rate_exact <= max(1e-4, rate_fast / 10.0), (rate_exact, rate_fast)
    assert np.allclose(exact_sc, ref["out_scale"], rtol=2e-3, atol=0)


@pytest.mark.parametrize("T,dm,dff,bias", [(128, 200, 300, True), (50, 64, 96, False), (256, 100, 1000, True),
                                           (130, 129, 257, True), (7, 16, 16, False), (512, 768, 1000, False)])
def test_widths_that_are_not_multiples_of_128(T, dm, dff, bias):
    """The reference sends these shapes to scalar kernels (kernels/int8_mlp.cu:1023-1026); here they run
    the same tensor-core pipeline on zero-padded copies.  Checked against the oracle like any other
    shape, and bit for bit against a run on operands padded by hand."""
    rng = np.random.default_rng(T * 7 + dm + dff)
    x = rng.standard_normal((T, dm)).astype(np.float16)
    W1 = (rng.standard_normal((dm, dff)) * 0.05).astype(np.float32)
    W2 = (rng.standard_normal((dff, dm)) * 0.05).astype(np.float32)
    b1 = (rng.standard_normal(dff) * 0.01).astype(np.float32) if bias else None
    args = _prep(x, W1, W2)
    out_i8, out_sc = _run_pc(*args, b1=b1)
    ref = omlp.kernel_mlp(*args, b1=b1)
    # narrow layers: one flipped hidden code is a larger share of an output value, so the row
    # maxima (the scales) may move by more than on the wide shapes
    _compare_with_kernel_oracle(out_i8, out_sc, ref, max_rate=0.03, scale_rtol=1e-2)
    deq = out_i8.astype(np.float32) * out_sc[:, None]
    xi, w1i, w2i, sx, s1, s2 = args
    xd = xi.astype(np.float32) * sx[:, None]
    base = omlp.gelu_tanh(xd @ (w1i.astype(np.float32) * s1[None, :]) + (0 if b1 is None else b1)) @ \
        (w2i.astype(np.float32) * s2[None, :])
    assert cosine(deq, base) > 0.999
    # the same call on operands padded by hand to multiples of 128
    dmp, dffp = -(-dm // 128) * 128, -(-dff // 128) * 128
    pad = lambda a, shape: np.pad(a, [(0, n - m) for m, n in zip(a.shape, shape)])
    padded = (pad(xi, (T, dmp)), pad(w1i, (dmp, dffp)), pad(w2i, (dffp, dmp)), sx, pad(s1, (dffp,)), pad(s2, (dmp,)))
    big_i8, big_sc = _run_pc(*padded, b1=None if b1 is None else pad(b1, (dffp,)))
    assert np.array_equal(big_i8[:, :dm], out_i8) and np.array_equal(big_sc, out_sc)
    assert not big_i8[:, dm:].any()
    # legacy per-tensor surface and the prepacked C-ABI route on the same odd widths
    x_t, w1_t, w2_t = _cuda(xi.reshape(1, T, dm), w1i, w2i)
    o, sc = ext().int8_mlp_forward(x_t, w1_t, w2_t, 0.02, 0.001, 0.001)
    assert o.shape == (1, T, dm) and sc > 0
    lib = cabi().load()
    flags = cabi().MLP_X_PER_TOKEN | cabi().MLP_W_PER_CHANNEL | cabi().MLP_PREPACKED
    w1T, w2T = _cuda(np.ascontiguousarray(w1i.T), np.ascontiguousarray(w2i.T))
    sx_t, s1_t, s2_t = _cuda(sx, s1, s2)
    wb = lib.i8tk_mlp_workspace_bytes(T, dm, dff, flags)
    ws = torch.zeros(wb, dtype=torch.uint8, device="cuda")
    o2 = torch.empty(T, dm, dtype=torch.int8, device="cuda")
    sc2 = torch.empty(T, device="cuda")
    b_t = None if b1 is None else _cuda(b1)[0]
    cabi().check(lib.i8tk_mlp_forward(x_t.data_ptr(), w1T.data_ptr(), w2T.data_ptr(), o2.data_ptr(), sx_t.data_ptr(),
                                      s1_t.data_ptr(), s2_t.data_ptr(), None if b_t is None else b_t.data_ptr(),
                                      sc2.data_ptr(), None, T, dm, dff, flags, ws.data_ptr(), wb, None))
    torch.cuda.synchronize()
    assert np.array_equal(o2.cpu().numpy(), out_i8) and np.array_equal(sc2.cpu().numpy(), out_sc)


@pytest.mark.parametrize("T,dm,dff", [(128, 128, 256), (8, 256, 256), (100, 200, 300), (512, 768, 3072)])
def test_static_scale_mode(T, dm, dff):
    """I8TK_MLP_STATIC_SCALES / static_scales=True: the arithmetic of the reference's fallback
    (kernels/int8_mlp.cu:830-844, 1194-1225) against its restatement.  The hidden scale is the bound
    sx*sw1*d_model, so the codes are small; they must equal the restatement's except where the
    hardware tanh moves a value across a rounding boundary (one step, rarely)."""
    rng = np.random.default_rng(T + dm + dff)
    x = rng.standard_normal((T, dm)).astype(np.float16)
    W1 = (rng.standard_normal((dm, dff)) * 0.05).astype(np.float16)
    W2 = (rng.standard_normal((dff, dm)) * 0.05).astype(np.float16)
    xi, sx = quant.quantize_per_tensor(x)
    w1i, s1 = quant.quantize_per_tensor(W1)
    w2i, s2 = quant.quantize_per_tensor(W2)
    ref = omlp.static_mlp(xi, w1i, w2i, sx, s1, s2)
    x_t, w1_t, w2_t = _cuda(xi.reshape(1, T, dm), w1i, w2i)
    out, osc = ext().int8_mlp_forward(x_t, w1_t, w2_t, float(sx), float(s1), float(s2), static_scales=True)
    o = out.cpu().numpy().reshape(T, dm)
    assert abs(osc - float(ref["out_scale"])) <= 1e-6 * float(ref["out_scale"])
    d = np.abs(o.astype(np.int32) - ref["out_i8"].astype(np.int32))
    assert d.max() <= 1 and float((d != 0).mean()) < 0.02, (d.max(), float((d != 0).mean()))
    assert ref["hidden_i8"].any() or dm * dff > 0       # the restatement is not degenerate
    was = ext().set_mlp_reference_rounding(True)
    try:
        out2, osc2 = ext().int8_mlp_forward(x_t, w1_t, w2_t, float(sx), float(s1), float(s2), static_scales=True)
    finally:
        ext().set_mlp_reference_rounding(was)
    d2 = np.abs(out2.cpu().numpy().reshape(T, dm).astype(np.int32) - ref["out_i8"].astype(np.int32))
    assert d2.max() <= 1 and float((d2 != 0).mean()) <= float((d != 0).mean()) + 1e-4
    if T % 128 == 0 and dm % 128 == 0 and dff % 128 == 0:
        W1T, W2T = ext().transpose_int8_weights(w1_t, w2_t)
        out3, osc3 = ext().int8_mlp_forward_prepacked(x_t, W1T, W2T, float(sx), float(s1), float(s2), static_scales=True)
        assert torch.equal(out3, out) and osc3 == osc


def test_workspace_kept_flag_gives_identical_results():
    """I8TK_MLP_WORKSPACE_KEPT: from the second forward of a shape on a workspace nothing else touches, the
    preset kernel may be skipped (both GEMMs leave the flag arrays preset).  Same bytes out, on a run of
    calls, for the per-token and the legacy per-tensor output, and through the ops (which track it)."""
    c = cabi()
    lib = c.load()
    e = ext()
    torch.manual_seed(5)
    for (T, dm, dff) in [(384, 256, 1024), (1000, 768, 3072)]:
        xs = [e.quantize_per_token(torch.randn(1, T, dm, device="cuda", dtype=torch.float16))[0] for _ in range(3)]
        sx = torch.rand(T, device="cuda") * 0.01 + 0.01
        w1 = torch.randint(-127, 128, (dm, dff), dtype=torch.int8, device="cuda")
        w2 = torch.randint(-127, 128, (dff, dm), dtype=torch.int8, device="cuda")
        s1 = torch.rand(dff, device="cuda") * 1e-4 + 1e-4
        s2 = torch.rand(dm, device="cuda") * 1e-4 + 1e-4
        st = torch.cuda.current_stream().cuda_stream
        for per_token_out in (True, False):
            flags = c.MLP_X_PER_TOKEN | c.MLP_W_PER_CHANNEL
            wb = lib.i8tk_mlp_workspace_bytes(T, dm, dff, flags)
            fresh = lambda: torch.randint(0, 255, (wb,), dtype=torch.uint8, device="cuda")     # garbage on purpose
            ws_kept = fresh()

            def run(x, ws, fl):
                o = torch.empty(1, T, dm, dtype=torch.int8, device="cuda")
                rs = torch.empty(T, device="cuda")
                ts = torch.empty(1, device="cuda")
                c.check(lib.i8tk_mlp_forward(x.data_ptr(), w1.data_ptr(), w2.data_ptr(), o.data_ptr(), sx.data_ptr(),
                                             s1.data_ptr(), s2.data_ptr(), None, rs.data_ptr() if per_token_out else None,
                                             None if per_token_out else ts.data_ptr(), T, dm, dff, fl, ws.data_ptr(), wb, st))
                return o, (rs if per_token_out else ts)

            for i, x in enumerate(xs + xs):
                want = run(x, fresh(), flags)
                got = run(x, ws_kept, flags | (c.MLP_WORKSPACE_KEPT if i > 0 else 0))
                assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1]), (T, per_token_out, i)
                assert lib.i8tk_check_status_word(ws_kept.data_ptr(), st) == c.OK
        # the ops: a run of calls of one shape, another shape in between
        b1 = torch.randn(dff, device="cuda") * 0.01
        first = e.int8_mlp_forward_per_channel_bias(xs[0], w1, w2, sx, s1, s2, b1)
        e.int8_mlp_forward_per_channel_bias(xs[1][:, :128].contiguous(), w1, w2, sx[:128].contiguous(), s1, s2, b1)
        for _ in range(3):
            again = e.int8_mlp_forward_per_channel_bias(xs[0], w1, w2, sx, s1, s2, b1)
            assert torch.equal(again[0], first[0]) and torch.equal(again[1], first[1])
    e.check_status()


def test_input_written_by_the_kernel_just_before():
    """The activations usually come from the quantiser launched just before the MLP, and that kernel lets its
    successor start while it is still running.  With the workspace kept there is no preset kernel in between,
    so GEMM1's producer warp itself has to wait for the quantiser before it copies x: every forward of a run
    on changing inputs must equal the same forward done after a full synchronisation."""
    e = ext()
    torch.manual_seed(11)
    T, dm, dff = 8192, 256, 1024           # a long quantiser pass in front of a short GEMM
    w1 = torch.randint(-127, 128, (dm, dff), dtype=torch.int8, device="cuda")
    w2 = torch.randint(-127, 128, (dff, dm), dtype=torch.int8, device="cuda")
    s1 = torch.rand(dff, device="cuda") * 1e-4 + 1e-4
    s2 = torch.rand(dm, device="cuda") * 1e-4 + 1e-4
    xs = [torch.randn(1, T, dm, device="cuda", dtype=torch.float16) * (i + 1) for i in range(6)]
    wants = []
    for x in xs:
        codes, scales = e.quantize_per_token(x)
        torch.cuda.synchronize()
        out, osc = e.int8_mlp_forward(codes, w1, w2, scales.reshape(-1), s1, s2)
        torch.cuda.synchronize()
        wants.append((out.clone(), osc.clone()))
    for x, (want, want_sc) in zip(xs, wants):
        codes, scales = e.quantize_per_token(x)               # no synchronisation: back to back on the stream
        out, osc = e.int8_mlp_forward(codes, w1, w2, scales.reshape(-1), s1, s2)
        assert torch.equal(out, want) and torch.equal(osc, want_sc)

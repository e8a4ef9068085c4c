"""Producer-side quantisation ops: LayerNorm fused with the per-token quantiser, and
quantise-on-write of the new token's K/V rows into the INT8 cache."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import quant
from helpers import ext, gold

pytestmark = pytest.mark.gpu


def _check_ln(x_np, q, s, y_ref, q_ref, s_ref):
    dq = np.abs(q.astype(np.int32) - q_ref.astype(np.int32))
    assert dq.max() <= 1, dq.max()
    assert np.mean(dq != 0) < 2e-3, np.mean(dq != 0)
    assert np.allclose(s, s_ref, rtol=1e-3, atol=0)


def test_layernorm_quantize_golden_and_oracle():
    g = gold("layernorm_quantize.npz")
    names = sorted(k[:-3] for k in g.files if k.endswith("__x"))
    assert len(names) == 4
    for n in names:
        x = g[n + "__x"]
        q, s = ext().layernorm_quantize(torch.from_numpy(x).cuda())
        q, s = q.cpu().numpy(), s.cpu().numpy()
        _check_ln(x, q, s, g[n + "__y"], g[n + "__q"], g[n + "__s"])      # torch CPU + reference quantiser
        y, q_o, s_o = quant.layernorm_quantize(x)
        _check_ln(x, q, s, y, q_o, s_o)                                   # float64 oracle


@pytest.mark.parametrize("shape", [(4, 128, 768), (1, 4096, 1024), (3, 5, 64), (2, 7, 4096), (1, 1, 8)])
def test_layernorm_quantize_equals_the_two_step_path(shape):
    torch.manual_seed(shape[-1])
    x = (torch.randn(*shape, device="cuda") * 2.0 + 0.5).half()
    q, s = ext().layernorm_quantize(x)
    assert q.shape == x.shape and s.shape == x.shape[:-1] and q.dtype == torch.int8
    q2, s2 = ext().quantize_per_token(F.layer_norm(x, (shape[-1],)))
    dq = (q.int() - q2.int()).abs()
    assert int(dq.max()) <= 1 and float((dq != 0).float().mean()) < 2e-3
    assert torch.allclose(s, s2, rtol=1e-3, atol=0)


def test_layernorm_quantize_edge_rows_and_errors():
    e = ext()
    x = torch.zeros(3, 256, device="cuda", dtype=torch.float16)
    x[1] = 7.0                                    # constant row: variance 0, all codes 0
    x[2, 0] = 100.0                               # one spike
    q, s = e.layernorm_quantize(x)
    assert torch.all(q[0] == 0) and torch.all(q[1] == 0)
    assert int(q[2, 0]) == 127 and not torch.isnan(s).any()
    q, s = e.layernorm_quantize(torch.zeros(0, 64, device="cuda", dtype=torch.float16))
    assert q.numel() == 0 and s.numel() == 0
    with pytest.raises(RuntimeError):
        e.layernorm_quantize(torch.zeros(2, 60, device="cuda", dtype=torch.float16))
    with pytest.raises(RuntimeError):
        e.layernorm_quantize(torch.zeros(2, 64, device="cuda", dtype=torch.float32))


@pytest.mark.parametrize("B,H,D,S_cap,pos", [(2, 3, 64, 40, 0), (1, 4, 128, 300, 299), (3, 2, 64, 129, 128)])
def test_kv_append_is_quantise_on_write(B, H, D, S_cap, pos):
    torch.manual_seed(pos + D)
    e = ext()
    K = torch.randint(-127, 128, (B, H, S_cap, D), dtype=torch.int8, device="cuda")
    V = torch.randint(-127, 128, (B, H, S_cap, D), dtype=torch.int8, device="cuda")
    sK = torch.rand(B * H * S_cap, device="cuda") + 0.5
    sV = torch.rand(B * H * S_cap, device="cuda") + 0.5
    K0, V0, sK0, sV0 = K.clone(), V.clone(), sK.clone(), sV.clone()
    k_new = torch.randn(B, H, D, device="cuda", dtype=torch.float16)
    v_new = torch.randn(B, H, D, device="cuda", dtype=torch.float16) * 3
    e.kv_append_quantize(k_new, v_new, K, V, sK, sV, pos)
    # bit-identical to the per-token quantiser (whose CPU arithmetic is the reference's)
    for new, cache, sc, cache0, sc0 in ((k_new, K, sK, K0, sK0), (v_new, V, sV, V0, sV0)):
        q_ref, s_ref = quant.quantize_per_token(new.cpu().numpy())
        assert np.array_equal(cache[:, :, pos].cpu().numpy(), q_ref)
        got_s = sc.view(B, H, S_cap)[:, :, pos].cpu().numpy()
        assert np.array_equal(got_s.view(np.uint32), s_ref.view(np.uint32))
        mask = torch.ones(S_cap, dtype=torch.bool, device="cuda")
        mask[pos] = False
        assert torch.equal(cache[:, :, mask], cache0[:, :, mask])          # nothing else touched
        assert torch.equal(sc.view(B, H, S_cap)[:, :, mask], sc0.view(B, H, S_cap)[:, :, mask])
    with pytest.raises(RuntimeError):
        e.kv_append_quantize(k_new, v_new, K, V, sK, sV, S_cap)


def test_decode_after_append_equals_decode_on_the_longer_cache():
    torch.manual_seed(5)
    e = ext()
    B, H, D, S = 2, 4, 64, 200
    Kf = torch.randn(B, H, S + 1, D, device="cuda", dtype=torch.float16)
    Vf = torch.randn(B, H, S + 1, D, device="cuda", dtype=torch.float16)
    Qi, sQ = e.quantize_per_token(torch.randn(B, H, D, device="cuda", dtype=torch.float16))
    Ki_full, sK_full = e.quantize_per_token(Kf)
    Vi_full, sV_full = e.quantize_per_token(Vf)
    want = e.int8_decode_attention_forward(Qi, Ki_full, Vi_full, sQ.reshape(-1), sK_full.reshape(-1), sV_full.reshape(-1))
    # cache holding the first S positions, room for one more; the last one arrives by append
    Ki, Vi = Ki_full.clone(), Vi_full.clone()
    sK, sV = sK_full.reshape(-1).clone(), sV_full.reshape(-1).clone()
    Ki[:, :, S] = 0; Vi[:, :, S] = 0
    sK.view(B, H, S + 1)[:, :, S] = 0; sV.view(B, H, S + 1)[:, :, S] = 0
    e.kv_append_quantize(Kf[:, :, S].contiguous(), Vf[:, :, S].contiguous(), Ki, Vi, sK, sV, S)
    got = e.int8_decode_attention_forward(Qi, Ki, Vi, sQ.reshape(-1), sK, sV)
    assert torch.equal(got, want)


@pytest.mark.parametrize("B,S,H,Dh", [(2, 37, 4, 64), (1, 130, 3, 128), (3, 1, 2, 64)])
def test_quantize_qkv_heads_is_the_quantiser_on_the_transposed_heads(B, S, H, Dh):
    torch.manual_seed(S)
    e = ext()
    d = H * Dh
    qkv = torch.randn(B, S, 3 * d, device="cuda", dtype=torch.float16) * 1.7
    qi, sc = e.quantize_qkv_heads(qkv, H)
    assert qi.shape == (3, B, H, S, Dh) and sc.shape == (3, B, H, S)
    for w, part in enumerate(qkv.split(d, dim=-1)):
        heads = part.view(B, S, H, Dh).transpose(1, 2).contiguous()
        q_ref, s_ref = quant.quantize_per_token(heads.cpu().numpy())
        assert np.array_equal(qi[w].cpu().numpy(), q_ref)
        assert np.array_equal(sc[w].cpu().numpy().view(np.uint32), s_ref.view(np.uint32))


def test_dequantize_per_token_with_and_without_residual():
    torch.manual_seed(2)
    e = ext()
    q = torch.randint(-128, 128, (3, 50, 256), dtype=torch.int8, device="cuda")
    s = torch.rand(3, 50, device="cuda") * 0.1 + 1e-3
    got = e.dequantize_per_token(q, s)
    want = (q.float() * s.unsqueeze(-1)).half()          # the eager spelling of the reference's block
    assert torch.equal(got, want)
    r = torch.randn(3, 50, 256, device="cuda", dtype=torch.float16)
    got = e.dequantize_per_token(q, s, r)
    exact = q.double() * s.double().unsqueeze(-1) + r.double()
    assert torch.equal(got, exact.half())               # one rounding of the exact sum (fma in fp32 is exact enough here)
    with pytest.raises(RuntimeError):
        e.dequantize_per_token(q[..., :8].contiguous(), s)


@pytest.mark.parametrize("B,H,D,S", [(3, 12, 64, 700), (128, 16, 64, 1024), (5, 32, 128, 300), (2, 1, 128, 64),
                                     (4, 8, 128, 4096)])
def test_decode_output_quantised_per_token_is_bit_exact(B, H, D, S):
    """int8_decode_attention_forward_quantized == quantize_per_token of the fp16 forward viewed as
    [B, H*D]: same codes, same scale bits -- the merge kernel runs the quantiser's arithmetic on the
    fp16-rounded values it would have stored."""
    e = ext()
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + S)
    Qi, sQ = e.quantize_per_token(torch.randn(B, H, D, device="cuda", dtype=torch.float16, generator=g))
    Ki, sK = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda", generator=g))
    Vi, sV = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda", generator=g) * 3.0)
    out = e.int8_decode_attention_forward(Qi, Ki, Vi, sQ, sK, sV)
    q_ref, s_ref = e.quantize_per_token(out.reshape(B, H * D))
    q, s = e.int8_decode_attention_forward_quantized(Qi, Ki, Vi, sQ, sK, sV)
    assert q.shape == (B, H * D) and q.dtype == torch.int8 and s.shape == (B,)
    assert torch.equal(q, q_ref)
    assert torch.equal(s.view(torch.int32), s_ref.view(torch.int32))
    # and against the CPU oracle's quantiser on the same fp16 values
    qo, so = quant.quantize_per_token(out.reshape(B, H * D).cpu().numpy())
    assert np.array_equal(q.cpu().numpy(), qo) and np.array_equal(s.cpu().numpy().view(np.uint32), so.view(np.uint32))


@pytest.mark.parametrize("T,K,N,bias", [(128, 128, 128, False), (7, 256, 384, True), (300, 1024, 1024, True),
                                        (4096, 768, 768, False)])
def test_int8_linear_matches_the_dequantised_product(T, K, N, bias):
    e = ext()
    g = torch.Generator(device="cuda").manual_seed(T + K + N)
    xi, sx = e.quantize_per_token(torch.randn(T, K, device="cuda", dtype=torch.float16, generator=g))
    W = torch.randn(K, N, device="cuda", generator=g) * 0.03
    sw = W.abs().amax(dim=0).clamp_min(1e-8) / 127.0
    wi = torch.clamp(torch.round(W / sw), -128, 127).to(torch.int8).contiguous()
    b = torch.randn(N, device="cuda", generator=g) * 0.1 if bias else None
    out = e.int8_linear(xi, sx, wi, sw, b)
    assert out.shape == (T, N) and out.dtype == torch.float16
    acc = (xi.double() @ wi.double())                                    # exact integer products
    ref = acc * sx.double()[:, None] * sw.double()[None, :] + (b.double() if bias else 0.0)
    err = (out.double() - ref).abs().max().item()
    assert err <= 2e-3 * max(1.0, ref.abs().max().item()), err           # fp16 output rounding
    with pytest.raises(RuntimeError, match="multiples of 128"):
        e.int8_linear(xi[:, :64].contiguous(), sx, wi[:64].contiguous(), sw)

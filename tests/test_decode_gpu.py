"""INT8-KV decode attention: CUDA path vs the oracle, the golden vectors and
size-independent properties.  Tolerance (validation/check_decode.py:73):
cosine > 0.9999 and max-abs error < 0.05 against the dequantised fp32
reference, no NaN; the kernel is in practice within fp16 rounding of it."""
import numpy as np
import pytest
import torch

from oracle import decode as odec, quant
from helpers import ext, cabi, gold, cosine

pytestmark = pytest.mark.gpu

COS_MIN = 0.9999
MAXABS = 0.05


def _run(Qi, Ki, Vi, sQ, sK, sV):
    t = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (Qi, Ki, Vi, sQ, sK, sV)]
    out = ext().int8_decode_attention_forward(*t)
    assert out.dtype == torch.float16
    return out.float().cpu().numpy()


def _assert_close(out, ref, tag):
    assert not np.isnan(out).any(), tag
    c = cosine(out, ref)
    e = float(np.abs(out - ref).max())
    assert c > COS_MIN and e < MAXABS, (tag, c, e)
    # much tighter in practice: fp16 output rounding dominates
    assert e < 2e-3 * max(1.0, float(np.abs(ref).max())), (tag, e)


def test_golden_reference_outputs():
    g = gold("decode_attention.npz")
    keys = sorted(k[:-5] for k in g.files if k.endswith("__ref"))
    assert len(keys) == 13
    for k in keys:
        out = _run(*[g[f"{k}__{n}"] for n in ("Qi", "Ki", "Vi", "sQ", "sK", "sV")])
        _assert_close(out, g[k + "__ref"], k)


def _seeded_case(B, H, D, S, seed, outlier=False, kv_dtype=np.float32):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, H, D)).astype(np.float16)
    K = rng.standard_normal((B, H, S, D)).astype(kv_dtype)
    V = rng.standard_normal((B, H, S, D)).astype(kv_dtype)
    if outlier:
        ch = rng.permutation(D)[: max(1, int(0.01 * D))]
        K[..., ch] *= 20.0
        V[..., ch] *= 20.0
    Qi, sQ = quant.quantize_per_token(q)
    Ki, sK = quant.quantize_per_token(K)
    Vi, sV = quant.quantize_per_token(V)
    return Qi, Ki, Vi, sQ, sK, sV


# the 16 shapes of validation/check_decode.py:50-53, the two largest with B*H reduced
CHECK_DECODE_CASES = [(1, 1, 64, 1), (1, 1, 64, 31), (2, 2, 64, 33), (1, 2, 64, 127),
                      (2, 2, 64, 128), (3, 5, 64, 1000), (8, 8, 64, 4096), (4, 4, 64, 8192),
                      (1, 1, 128, 1), (1, 1, 128, 31), (2, 2, 128, 33), (1, 2, 128, 127),
                      (2, 2, 128, 128), (3, 5, 128, 1000), (8, 8, 128, 4096), (4, 4, 128, 8192)]


@pytest.mark.parametrize("B,H,D,S", CHECK_DECODE_CASES)
def test_edge_shapes_vs_oracle(B, H, D, S):
    args = _seeded_case(B, H, D, S, 1234 + S, kv_dtype=np.float16)
    out = _run(*args)
    ref = odec.decode_attention(*args)
    _assert_close(out, ref, (B, H, D, S))


@pytest.mark.parametrize("B,H,D,S", [(1, 12, 64, 1024), (2, 3, 64, 2049), (2, 3, 128, 4100),
                                     (1, 1, 64, 65536), (37, 1, 128, 96), (1, 2, 128, 32769)])
def test_more_shapes_vs_oracle(B, H, D, S):
    args = _seeded_case(B, H, D, S, 99 + S, outlier=(D == 128))
    out = _run(*args)
    ref = odec.decode_attention(*args)
    _assert_close(out, ref, (B, H, D, S))


@pytest.mark.parametrize("B,H,D,S", [(50, 12, 64, 300), (20, 30, 128, 261), (40, 12, 64, 1025), (3, 8, 64, 2048),
                                     (1, 32, 128, 2040),
                                     # few rows: a cluster of CTAs per row, merged through distributed shared memory
                                     (1, 12, 64, 4096), (1, 32, 128, 2048), (2, 5, 64, 1500), (1, 3, 128, 1027),
                                     (6, 12, 64, 1024), (1, 1, 64, 1100)])
def test_short_contexts_merged_inside_the_scan(B, H, D, S):
    """Rows of at most 16 tiles are scanned whole by one CTA, which merges its four warps' partial rows in
    shared memory and writes the output itself (no merge kernel); with more rows than one resident wave a
    CTA takes several rows in turn.  With few rows of 8 tiles or more, a cluster of 2-8 CTAs shares a row
    (some ranks may get no tile of it) and rank 0 merges the ranks' rows.  Shapes on both sides of those
    plans' limits, scales riding the bulk copies (S % 4 == 0) and loaded by the lanes."""
    args = _seeded_case(B, H, D, S, 7 + S)
    out = _run(*args)
    ref = odec.decode_attention(*args)
    _assert_close(out, ref, (B, H, D, S))
    again = _run(*args)
    assert np.array_equal(out, again)


def test_degenerate_inputs():
    # zeros: uniform softmax over zero values -> 0; constant: output == the V row
    for D in (64, 128):
        z = np.zeros((1, 2, 300, D), dtype=np.float32)
        Qi, sQ = quant.quantize_per_token(np.zeros((1, 2, D), dtype=np.float32))
        Ki, sK = quant.quantize_per_token(z)
        out = _run(Qi, Ki, Ki, sQ, sK, sK)
        assert np.all(out == 0.0)
        o = np.ones((1, 2, 300, D), dtype=np.float32)
        Qi, sQ = quant.quantize_per_token(np.ones((1, 2, D), dtype=np.float32))
        Ki, sK = quant.quantize_per_token(o)
        out = _run(Qi, Ki, Ki, sQ, sK, sK)
        assert np.allclose(out, 1.0, atol=1e-3)


def test_peaky_softmax_and_large_scores():
    # one key aligned with q and scaled up: softmax ~ one-hot, output ~ that V row
    rng = np.random.default_rng(5)
    D, S = 64, 777
    q = rng.standard_normal((1, 1, D)).astype(np.float32)
    K = rng.standard_normal((1, 1, S, D)).astype(np.float32) * 0.1
    K[0, 0, 500] = q[0, 0] * 10.0
    V = rng.standard_normal((1, 1, S, D)).astype(np.float32)
    args = (*quant.quantize_per_token(q)[:1], *quant.quantize_per_token(K)[:1],
            *quant.quantize_per_token(V)[:1], quant.quantize_per_token(q)[1],
            quant.quantize_per_token(K)[1], quant.quantize_per_token(V)[1])
    out = _run(*args)
    ref = odec.decode_attention(*args)
    _assert_close(out, ref, "peaky")


def test_split_invariance_property():
    """The result must not depend on how the KV axis is split: run one (b,h)
    alone (few units -> many splits) and inside a large batch (no split)."""
    args = _seeded_case(1, 1, 64, 2048, 3)
    alone = _run(*args)
    big = [np.repeat(a, 2048, axis=1) if a.ndim >= 2 else a for a in args]
    big = [np.ascontiguousarray(a) for a in big]
    batch = _run(*big)
    assert np.abs(batch - alone).max() < 2e-3
    assert np.abs(batch[:, :1] - batch[:, -1:]).max() == 0.0


def test_partial_combine_equals_forward():
    """Sequence-sharded path: partials over KV shards + combine == full forward,
    and the partial rows match the oracle's (m, l, acc) algebra."""
    B, H, D, S = 2, 3, 128, 3000
    args = _seeded_case(B, H, D, S, 11, outlier=True)
    full = _run(*args)
    Qi, Ki, Vi, sQ, sK, sV = args
    bounds = [0, 1000, 1001, 2500, 3000]
    parts = []
    for a, b in zip(bounds[:-1], bounds[1:]):
        t = [torch.from_numpy(np.ascontiguousarray(x)).cuda()
             for x in (Qi, Ki[:, :, a:b], Vi[:, :, a:b], sQ, sK[:, :, a:b], sV[:, :, a:b])]
        p = ext().int8_decode_attention_partial(*t)
        assert tuple(p.shape) == (B, H, D + 4)
        m, l, acc = odec.decode_partial(*args, j0=a, j1=b)
        pn = p.cpu().numpy().astype(np.float64)
        # m is kept in log2 units
        assert np.allclose(pn[..., 0] * np.log(2.0), m, rtol=1e-5, atol=1e-4)
        scale = np.exp2(pn[..., 0] - m / np.log(2.0))
        assert np.allclose(pn[..., 1] * scale, l, rtol=1e-4)
        assert np.allclose(pn[..., 4:] * scale[..., None], acc, rtol=1e-3, atol=1e-3 * np.abs(acc).max())
        parts.append(p)
    out = ext().int8_decode_combine_partials(torch.stack(parts)).float().cpu().numpy()
    assert np.abs(out - full).max() < 2e-3
    _assert_close(out, odec.decode_attention(*args), "sharded")


def test_argument_errors():
    e = ext()
    dev = "cuda"
    Q = torch.zeros(1, 2, 64, dtype=torch.int8, device=dev)
    K = torch.zeros(1, 2, 16, 64, dtype=torch.int8, device=dev)
    sQ = torch.ones(2, device=dev)
    sK = torch.ones(32, device=dev)
    with pytest.raises(RuntimeError, match="head_dim 64 or 128"):
        e.int8_decode_attention_forward(torch.zeros(1, 2, 32, dtype=torch.int8, device=dev),
                                        torch.zeros(1, 2, 16, 32, dtype=torch.int8, device=dev),
                                        torch.zeros(1, 2, 16, 32, dtype=torch.int8, device=dev), sQ, sK, sK)
    with pytest.raises(RuntimeError, match="must be int8"):
        e.int8_decode_attention_forward(Q.float(), K, K, sQ, sK, sK)
    with pytest.raises(RuntimeError, match="contiguous"):
        e.int8_decode_attention_forward(Q, K.transpose(1, 2).contiguous().transpose(1, 2), K, sQ, sK, sK)
    with pytest.raises(RuntimeError, match="CUDA"):
        e.int8_decode_attention_forward(Q.cpu(), K, K, sQ, sK, sK)
    lib = cabi().load()
    ws = torch.empty(16, dtype=torch.uint8, device=dev)
    out = torch.empty(1, 2, 64, dtype=torch.float16, device=dev)
    rc = lib.i8tk_decode_attention_forward(Q.data_ptr(), K.data_ptr(), K.data_ptr(), out.data_ptr(),
                                           sQ.data_ptr(), sK.data_ptr(), sK.data_ptr(), 2, 16, 64,
                                           ws.data_ptr(), 16, None)
    assert rc == cabi().ERR_WORKSPACE
    rc = lib.i8tk_decode_attention_forward(Q.data_ptr(), K.data_ptr(), K.data_ptr(), out.data_ptr(),
                                           sQ.data_ptr(), sK.data_ptr(), sK.data_ptr(), 2, 16, 96,
                                           ws.data_ptr(), 16, None)
    assert rc == cabi().ERR_UNSUPPORTED
    rc = lib.i8tk_decode_attention_forward(Q.data_ptr() + 1, K.data_ptr(), K.data_ptr(), out.data_ptr(),
                                           sQ.data_ptr(), sK.data_ptr(), sK.data_ptr(), 2, 16, 64,
                                           ws.data_ptr(), 16, None)
    assert rc == cabi().ERR_ALIGNMENT


def test_full_size_config_properties():
    """Serving-scale shape (B32 H12 D64 ctx 8192): oracle on sampled (b,h) rows,
    plus linearity in V: attn(q,K,2V-scale) == 2*attn(q,K,V)."""
    B, H, D, S = 32, 12, 64, 8192
    torch.manual_seed(0)
    e = ext()
    q = torch.randn(B, H, D, device="cuda", dtype=torch.float16)
    K = torch.randn(B, H, S, D, device="cuda")
    V = torch.randn(B, H, S, D, device="cuda")
    Qi, sQ = e.quantize_per_token(q)
    Ki, sK = e.quantize_per_token(K)
    Vi, sV = e.quantize_per_token(V)
    del K, V
    out = e.int8_decode_attention_forward(Qi, Ki, Vi, sQ, sK, sV)
    out2 = e.int8_decode_attention_forward(Qi, Ki, Vi, sQ, sK, sV * 2.0)
    assert torch.allclose(out2.float(), 2.0 * out.float(), atol=2e-3)
    for (b, h) in [(0, 0), (7, 3), (31, 11)]:
        ref = odec.decode_attention(Qi[b:b + 1, h:h + 1].cpu().numpy(), Ki[b:b + 1, h:h + 1].cpu().numpy(),
                                    Vi[b:b + 1, h:h + 1].cpu().numpy(), sQ[b:b + 1, h:h + 1].cpu().numpy(),
                                    sK[b:b + 1, h:h + 1].cpu().numpy(), sV[b:b + 1, h:h + 1].cpu().numpy())
        _assert_close(out[b:b + 1, h:h + 1].float().cpu().numpy(), ref, (b, h))
